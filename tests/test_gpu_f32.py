"""fp32 kernels (GEMM, GEMV, general / 1x1 / Winograd Conv2D, depthwise) against the CPU
oracle.  Two tolerances are asserted for every comparison: the reference's element-wise form
|got - ref| <= abs_err + rel_err * |ref| (ExpectTensorNear,
test/ccutils/mace/ops/testing/test_utils.h:208-233) with rel_err = 1e-4 (Winograd: 1e-3 against
the DIRECT fp32 convolution, as the 3x3 Winograd path is specified) and abs_err = rel_err *
rms(ref), and the range-normalised max |got - ref| <= tol * max |ref|.  Plus the reference's own
literal known-answer cases."""
import numpy as np
import pytest

from helpers import near_ratio

pytestmark = pytest.mark.gpu
PAD = {"VALID": 0, "SAME": 1, "FULL": 2}


@pytest.fixture(scope="module")
def ctx():
    import mace_b200
    c = mace_b200.Context(0)
    yield c
    c.close()


WORST = {}  # label -> (element-wise ratio, range-normalised error), printed by the last test


def rel_err(got, ref, tol=None, label=None):
    """Range-normalised error; with tol also asserts the element-wise form at rel_err = tol."""
    rng_err = float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))
    if tol is not None:
        ratio = near_ratio(got, ref, tol)
        if label:
            prev = WORST.get(label, (0.0, 0.0))
            WORST[label] = (max(prev[0], ratio), max(prev[1], rng_err))
        assert ratio <= 1.0, "element-wise |got - ref| <= %g * (rms + |ref|) violated: ratio %.3f" % (tol, ratio)
    return rng_err


@pytest.mark.parametrize("maj", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 0), (0, 0, 1), (1, 1, 1)])
@pytest.mark.parametrize("shape", [(1, 5, 5, 5), (2, 47, 61, 33), (3, 64, 128, 96), (1, 1, 300, 700)])
def test_gemm_f32(ctx, orc, maj, shape):
    """Major-order combinations of test/ccunit/mace/ops/arm/fp32/gemm_test.cc:28-121."""
    batch, M, N, K = shape
    rng = np.random.Generator(np.random.PCG64(M + N))
    A = rng.standard_normal((batch, M, K)).astype(np.float32)
    B = rng.standard_normal((batch, K, N)).astype(np.float32)
    A_st = np.ascontiguousarray(np.swapaxes(A, 1, 2)) if maj[0] else A
    B_st = np.ascontiguousarray(np.swapaxes(B, 1, 2)) if maj[1] else B
    dA, dB, dC = ctx.upload(A_st), ctx.upload(B_st), ctx.alloc(batch * M * N * 4)
    ctx.gemm_f32(dA, dB, dC, batch, M, N, K, bool(maj[0]), bool(maj[1]), bool(maj[2]))
    got = ctx.download(dC, (batch * M * N,), np.float32)
    ref = orc.gemm_f32(A_st, B_st, batch, M, N, K, bool(maj[0]), bool(maj[1]), bool(maj[2]))
    assert rel_err(got, ref, 1e-4, "gemm_f32") <= 1e-4
    for b in (dA, dB, dC):
        b.free()


@pytest.mark.parametrize("shape", [(3, 64, 3200, 64), (1, 200, 1000, 40), (2, 24, 132, 260),
                                   (1, 300, 4100, 512)])
def test_gemm_f32_tensor_core(ctx, orc, shape):
    """Row-major A, B and C with 16-byte aligned rows run on the tensor cores (tf32 MMAs on
    hi/lo split operands); ragged M, N and K tails, with values of mixed magnitude."""
    batch, M, N, K = shape
    rng = np.random.Generator(np.random.PCG64(K))
    A = (rng.standard_normal((batch, M, K)) * np.exp(rng.uniform(-3, 3, (batch, M, K)))).astype(np.float32)
    B = rng.standard_normal((batch, K, N)).astype(np.float32)
    dA, dB, dC = ctx.upload(A), ctx.upload(B), ctx.alloc(batch * M * N * 4)
    before = ctx.launches_tensor_core
    ctx.gemm_f32(dA, dB, dC, batch, M, N, K)
    assert ctx.launches_tensor_core == before + 1, "tensor-core kernel did not run"
    got = ctx.download(dC, (batch * M * N,), np.float32)
    ref = orc.gemm_f32(A, B, batch, M, N, K)
    assert rel_err(got, ref, 1e-4, "gemm_f32_tensor_core") <= 1e-5  # element-wise at the specified 1e-4
    for b in (dA, dB, dC):
        b.free()


def test_gemm_f32_literals_and_one_side_batched(ctx, orc):
    a = np.arange(1, 7, dtype=np.float32)  # matmul_test.cc:55-58
    dA, dC = ctx.upload(a), ctx.alloc(16)
    ctx.gemm_f32(dA, dA, dC, 1, 2, 2, 3)
    assert ctx.download(dC, (4,), np.float32).tolist() == [22, 28, 49, 64]
    rng = np.random.Generator(np.random.PCG64(3))
    A = rng.standard_normal((1, 24, 40)).astype(np.float32)
    B = rng.standard_normal((4, 40, 56)).astype(np.float32)
    dA, dB, dC = ctx.upload(A), ctx.upload(B), ctx.alloc(4 * 24 * 56 * 4)
    ctx.gemm_f32(dA, dB, dC, 4, 24, 56, 40, a_batched=False)
    ref = orc.gemm_f32(A, B, 4, 24, 56, 40, a_batched=False)
    assert rel_err(ctx.download(dC, (4 * 24 * 56,), np.float32), ref, 1e-4, "gemm_f32") <= 1e-4


@pytest.mark.parametrize("shape", [(1, 16, 4), (3, 63, 257), (17, 65, 100), (36, 50, 260), (256, 1000, 2048)])
def test_gemv_f32(ctx, orc, shape):
    batch, rows, K = shape
    rng = np.random.Generator(np.random.PCG64(7))
    lhs = rng.standard_normal((rows, K)).astype(np.float32)
    rhs = rng.standard_normal((batch, K)).astype(np.float32)
    bias = rng.standard_normal(rows).astype(np.float32)
    dl, dr, db, do = ctx.upload(lhs), ctx.upload(rhs), ctx.upload(bias), ctx.alloc(batch * rows * 4)
    ctx.gemv_f32(dl, dr, db, do, batch, rows, K)
    ref = orc.gemv_f32(lhs, rhs, bias, batch, rows, K)
    assert rel_err(ctx.download(do, (batch * rows,), np.float32), ref, 1e-4, "gemv_f32") <= 1e-4


def _conv_inputs(shape, fshape, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.random(shape, dtype=np.float32)
    fan_in = fshape[1] * fshape[2] * fshape[3]
    f = (rng.standard_normal(fshape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    bias = (rng.standard_normal(fshape[0]) * 0.01).astype(np.float32)
    return x, f, bias


@pytest.mark.parametrize("case", [
    # N, C, H, W, O, KH, KW, stride, dilation, padding, activation
    (1, 2, 3, 3, 1, 3, 3, 1, 1, "VALID", 0),
    (2, 16, 14, 14, 32, 1, 1, 1, 1, "VALID", 1),      # 1x1 -> batched GEMM
    (1, 3, 33, 35, 8, 7, 7, 2, 1, "SAME", 1),         # ResNet-style 7x7 stride-2 stem
    (2, 8, 15, 15, 16, 1, 1, 2, 1, "SAME", 0),        # 1x1 stride 2
    (1, 4, 12, 13, 6, 3, 3, 1, 2, "SAME", 2),         # dilated, RELUX
    (1, 5, 9, 9, 7, 5, 5, 1, 1, "FULL", 6),           # LEAKYRELU
])
def test_conv2d_f32(ctx, orc, case):
    N, C, H, W, O, KH, KW, st, dil, padding, act = case
    x, f, bias = _conv_inputs((N, C, H, W), (O, C, KH, KW), H * 3 + C)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, KH, KW, (dil, dil), (st, st), PAD[padding])
    ref = orc.conv2d_f32(x, f, bias, (st, st), (dil, dil), (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.1)
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(ref.nbytes)
    ctx.conv2d_f32(dx, df, db, do, N, C, H, W, O, KH, KW, (st, st), (dil, dil), (ph >> 1, pw >> 1),
                   (Ho, Wo), act, 0.5, 0.1)
    assert rel_err(ctx.download(do, ref.shape, np.float32), ref, 1e-4, "conv2d_f32") <= 1e-4


def test_conv2d_f32_reference_literals(ctx, kats):
    """TestNHWCSimple3x3VALID / SAME: all-ones 3x3x2 input and filter, bias 0.1 -> 18.1 ..."""
    for name in ("conv2d_f32_3x3_valid", "conv2d_f32_3x3_same"):
        k = kats[name]
        x = np.ones((1, 2, 3, 3), np.float32)
        f = np.ones((1, 2, 3, 3), np.float32)
        bias = np.array(k["bias"], np.float32)
        same = k["padding"] == "SAME"
        Ho = 3 if same else 1
        pad = (1, 1) if same else (0, 0)
        exp = np.array(k["expected"], np.float32).reshape(1, 1, Ho, Ho)
        dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(exp.nbytes)
        ctx.conv2d_f32(dx, df, db, do, 1, 2, 3, 3, 1, 3, 3, (1, 1), (1, 1), pad, (Ho, Ho))
        np.testing.assert_allclose(ctx.download(do, exp.shape, np.float32), exp, rtol=1e-5)
        for tile in (2, 6):
            ctx.winograd_f32(dx, df, db, do, 1, 2, 3, 3, 1, pad, (Ho, Ho), tile=tile)
            np.testing.assert_allclose(ctx.download(do, exp.shape, np.float32), exp, rtol=1e-4)


@pytest.mark.parametrize("case", [
    # N, C, H, W, O, padding, activation
    (1, 8, 9, 9, 8, "SAME", 0),        # small input -> F(2,3)
    (2, 16, 14, 17, 24, "VALID", 1),
    (1, 8, 20, 20, 16, "SAME", 0),     # larger than 16x16 -> F(6,3)
    (2, 64, 56, 56, 64, "SAME", 1),    # config-1 shape, reduced batch
    (1, 32, 31, 29, 40, "VALID", 2),   # tile tails
])
def test_winograd_f32(ctx, orc, case):
    N, C, H, W, O, padding, act = case
    x, f, bias = _conv_inputs((N, C, H, W), (O, C, 3, 3), H + C)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (1, 1), PAD[padding])
    direct = orc.conv2d_f32(x, f, bias, (1, 1), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.0)
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(direct.nbytes)
    ctx.winograd_f32(dx, df, db, do, N, C, H, W, O, (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.0)
    got = ctx.download(do, direct.shape, np.float32)
    assert rel_err(got, direct, 1e-3, "winograd_vs_direct") <= 1e-3
    # against the oracle's Winograd restatement (same algorithm, same tile rule): tighter
    wino = orc.winograd_f32(x, f, bias, (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.0)
    assert rel_err(got, wino, 1e-4, "winograd_vs_oracle_winograd") <= 1e-4
    # cached transformed filter gives the same result
    tile = 6 if (H > 16 and W > 16) else 2
    dU = ctx.alloc((tile + 2) ** 2 * O * C * 4)
    ctx.winograd_transform_filter(df, dU, C, O, tile)
    ctx.winograd_f32(dx, None, db, do, N, C, H, W, O, (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.0,
                     transformed=dU)
    assert np.array_equal(ctx.download(do, direct.shape, np.float32), got)
    # the one-thread-per-tile output transform computes the same values as the plane-at-a-time one
    ctx.set_option("wino_plane", 0)
    try:
        ctx.winograd_f32(dx, df, db, do, N, C, H, W, O, (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.0)
    finally:
        ctx.set_option("wino_plane", 1)
    assert np.array_equal(ctx.download(do, direct.shape, np.float32), got)


def test_dwconv_f32(ctx, orc, kats):
    k = kats["dwconv_f32_2x2_valid"]  # SimpleValidTest, depthwise_conv2d_test.cc:26-84
    x = np.transpose(np.array(k["input"], np.float32).reshape(1, 3, 3, 2), (0, 3, 1, 2)).copy()
    f = np.array(k["filter"], np.float32).reshape(1, 2, 2, 2)
    bias = np.array(k["bias"], np.float32)
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(8 * 4)
    ctx.dwconv_f32(dx, df, db, do, 1, 2, 3, 3, 1, 2, 2, (1, 1), (1, 1), (0, 0), (2, 2))
    got = np.transpose(ctx.download(do, (1, 2, 2, 2), np.float32), (0, 2, 3, 1))
    np.testing.assert_allclose(got.ravel(), np.array(k["expected"], np.float32), rtol=1e-5)
    rng = np.random.Generator(np.random.PCG64(1))
    x = rng.standard_normal((2, 12, 17, 15)).astype(np.float32)
    f = rng.standard_normal((2, 12, 3, 3)).astype(np.float32)
    bias = rng.standard_normal(24).astype(np.float32)
    ref = orc.dwconv_f32(x, f, bias, (2, 2), (1, 1), (0, 0), (9, 8), 1)
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(ref.nbytes)
    ctx.dwconv_f32(dx, df, db, do, 2, 12, 17, 15, 2, 3, 3, (2, 2), (1, 1), (0, 0), (9, 8), 1)
    assert rel_err(ctx.download(do, ref.shape, np.float32), ref, 1e-4, "dwconv_f32") <= 1e-4


def test_winograd_config1_full_size(ctx, orc):
    """Input [32,64,56,56], filter [64,64,3,3], SAME (the full configuration): every image against the oracle's direct convolution (threaded, a few seconds), and one
    image of the batch-32 call against the same image run alone (the batch entries are independent)."""
    N, C, H, W, O = 32, 64, 56, 56, 64
    rng = np.random.Generator(np.random.PCG64(0))
    x = rng.random((N, C, H, W), dtype=np.float32)
    f = (rng.standard_normal((O, C, 3, 3)) * np.sqrt(2.0 / (9 * C))).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.01).astype(np.float32)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(N * O * H * W * 4)
    ctx.winograd_f32(dx, df, db, do, N, C, H, W, O, (1, 1), (H, W))
    got = ctx.download(do, (N, O, H, W), np.float32)
    ref = orc.conv2d_f32(x, f, bias, (1, 1), (1, 1), (1, 1), (H, W), 0, 0.0, 0.0)  # all 32 images
    assert rel_err(got, ref, 1e-3, "winograd_config1_vs_direct") <= 1e-3
    d1, o1 = ctx.upload(x[17:18]), ctx.alloc(O * H * W * 4)
    ctx.winograd_f32(d1, df, db, o1, 1, C, H, W, O, (1, 1), (H, W))
    alone = ctx.download(o1, (1, O, H, W), np.float32)
    assert np.array_equal(alone[0], got[17])


@pytest.mark.parametrize("case", [
    # N, C, H, W, O, KH, KW, stride, dilation, padding, activation
    (3, 3, 64, 64, 64, 7, 7, 2, 1, "SAME", 1),     # stem shape: K = 147 (filter rows repacked), 1024 positions
    (2, 64, 30, 30, 48, 1, 1, 2, 1, "SAME", 0),    # 1x1 stride 2: 225 positions -> images merged
    (5, 96, 7, 7, 40, 1, 1, 1, 1, "VALID", 1),     # 1x1 stride 1 with 49 positions -> images merged
    (2, 32, 20, 24, 24, 3, 3, 2, 1, "SAME", 6),    # 3x3 stride 2: 120 positions -> merged
    (2, 16, 40, 40, 32, 3, 3, 1, 2, "SAME", 2),    # dilated 3x3, 1600 positions per image
    (1, 8, 33, 47, 16, 5, 3, 1, 1, "FULL", 0),     # ragged everything
])
@pytest.mark.parametrize("budget_mb", [1024, 1])
def test_conv2d_f32_column_route(ctx, orc, case, budget_mb):
    """General convolutions large enough for the im2col + tensor-core GEMM route, with the
    column matrix in one piece and split into chunks of images (1 MiB budget)."""
    N, C, H, W, O, KH, KW, st, dil, padding, act = case
    x, f, bias = _conv_inputs((N, C, H, W), (O, C, KH, KW), H * 5 + C)
    x = x * 2 - 1
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, KH, KW, (dil, dil), (st, st), PAD[padding])
    ref = orc.conv2d_f32(x, f, bias, (st, st), (dil, dil), (ph >> 1, pw >> 1), (Ho, Wo), act, 0.5, 0.1)
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(ref.nbytes)
    ctx.set_option("col_budget_mb", budget_mb)
    before = ctx.launches_tensor_core
    try:
        ctx.conv2d_f32(dx, df, db, do, N, C, H, W, O, KH, KW, (st, st), (dil, dil), (ph >> 1, pw >> 1),
                       (Ho, Wo), act, 0.5, 0.1)
    finally:
        ctx.set_option("col_budget_mb", 1024)
    assert ctx.launches_tensor_core > before, "tensor-core GEMM did not run"
    assert rel_err(ctx.download(do, ref.shape, np.float32), ref, 1e-4, "conv2d_f32_column_route") <= 1e-4
    for b in (dx, df, db, do):
        b.free()


@pytest.mark.parametrize("case", [
    # N, C, H, W, kernel, stride, dilation, padding
    (2, 5, 17, 19, 3, 2, 1, "SAME"),      # ResNet's 3x3 stride-2 max pool
    (1, 3, 8, 8, 2, 2, 1, "VALID"),
    (2, 16, 7, 7, 7, 1, 1, "VALID"),      # global pooling
    (1, 4, 13, 11, 3, 1, 2, "SAME"),      # dilated
    (2, 3, 10, 10, 5, 3, 1, "FULL"),      # windows that overlap the border by more than half
    (2, 6, 16, 24, 3, 2, 1, "SAME"),      # rows of a multiple of 4: four outputs per thread, 128-bit accesses
    (1, 3, 20, 20, 3, 2, 1, "VALID"),     # ... with an output width that is not a multiple of 4
    (2, 4, 112, 112, 3, 2, 1, "SAME"),    # ResNet's pooling layer at full size
])
@pytest.mark.parametrize("ptype", [1, 2])
def test_pooling_f32(ctx, orc, case, ptype):
    N, C, H, W, k, st, dil, padding = case
    rng = np.random.Generator(np.random.PCG64(H + ptype))
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, k, k, (dil, dil), (st, st), PAD[padding])
    ref = orc.pooling_f32(x, (k, k), (st, st), (dil, dil), (ph >> 1, pw >> 1), (Ho, Wo), ptype)
    dx, do = ctx.upload(x), ctx.alloc(ref.nbytes)
    ctx.pooling_f32(dx, do, N, C, H, W, (k, k), (st, st), (dil, dil), (ph >> 1, pw >> 1), (Ho, Wo), ptype)
    got = ctx.download(do, ref.shape, np.float32)
    if ptype == 2:
        assert np.array_equal(got, ref)          # a maximum has no rounding
    else:
        assert rel_err(got, ref, 1e-6, "pooling_f32") <= 1e-6
    dx.free(); do.free()


def test_pooling_f32_reference_literals(ctx):
    """PoolingOpTest.MAX_VALID / AVG_VALID (test/ccunit/mace/ops/pooling_test.cc:27-61, 301-336)."""
    x = np.ascontiguousarray(np.arange(32, dtype=np.float32).reshape(1, 2, 4, 4))
    dx, do = ctx.upload(x), ctx.alloc(8 * 4)
    ctx.pooling_f32(dx, do, 1, 2, 4, 4, (2, 2), (2, 2), (1, 1), (0, 0), (2, 2), 2)
    assert ctx.download(do, (8,), np.float32).tolist() == [5, 7, 13, 15, 21, 23, 29, 31]
    ctx.pooling_f32(dx, do, 1, 2, 4, 4, (2, 2), (2, 2), (1, 1), (0, 0), (2, 2), 1)
    assert ctx.download(do, (8,), np.float32).tolist() == [2.5, 4.5, 10.5, 12.5, 18.5, 20.5, 26.5, 28.5]


@pytest.mark.parametrize("size", [1, 6, 1000, 4099, 1 << 20])
def test_eltwise_f32(ctx, orc, size):
    """Same-shape and tensor-scalar forms; the results are single IEEE operations (or two
    products and a sum), so they must be bit-identical to the CPU's."""
    rng = np.random.Generator(np.random.PCG64(size))
    a = rng.standard_normal(size).astype(np.float32)
    b = (rng.standard_normal(size) + 2.5).astype(np.float32)
    da, db, do = ctx.upload(a), ctx.upload(b), ctx.alloc(size * 4)
    for type_ in (0, 1, 2, 3, 4, 5, 6, 7, 8):
        for swapped in (False, True):
            ctx.eltwise_f32(da, db, do, size, type_, swapped=swapped)
            assert np.array_equal(ctx.download(do, (size,), np.float32),
                                  orc.eltwise_f32(a, b, type_, swapped=swapped)), (type_, swapped)
            ctx.eltwise_f32(da, None, do, size, type_, swapped=swapped, scalar=0.75)
            assert np.array_equal(ctx.download(do, (size,), np.float32),
                                  orc.eltwise_f32(a, None, type_, swapped=swapped, scalar=0.75)), type_
    for swapped in (False, True):
        ctx.eltwise_f32(da, db, do, size, 0, coeff=(0.3, -1.7), swapped=swapped)
        assert np.array_equal(ctx.download(do, (size,), np.float32),
                              orc.eltwise_f32(a, b, 0, coeff=(0.3, -1.7), swapped=swapped))
    ctx.eltwise_f32(da, None, do, size, 12, coeff=(-0.5, 0.25))
    assert np.array_equal(ctx.download(do, (size,), np.float32), orc.eltwise_f32(a, None, 12, coeff=(-0.5, 0.25)))
    import mace_b200
    with pytest.raises(mace_b200.MaceB200Error):
        ctx.eltwise_f32(da, db, do, size, 9)           # POW is not built
    with pytest.raises(mace_b200.MaceB200Error):
        ctx.eltwise_f32(da, None, do, size, 12, coeff=(1.0, 0.0))   # Clip needs min < max
    for buf in (da, db, do):
        buf.free()


@pytest.mark.parametrize("act", [0, 1, 2, 6])
def test_activation_f32(ctx, orc, act):
    rng = np.random.Generator(np.random.PCG64(act))
    x = (rng.standard_normal(100003) * 3).astype(np.float32)
    dx, do = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.activation_f32(dx, do, x.size, act, 2.0, 0.1)
    assert rel_err(ctx.download(do, x.shape, np.float32), orc.activation_f32(x, act, 2.0, 0.1), 1e-7, "activation") <= 1e-7
    ctx.activation_f32(dx, dx, x.size, act, 2.0, 0.1)   # in place
    assert rel_err(ctx.download(dx, x.shape, np.float32), orc.activation_f32(x, act, 2.0, 0.1), 1e-7, "activation") <= 1e-7
    dx.free(); do.free()


@pytest.mark.parametrize("shape", [(2, 4, 1), (3, 1001, 1), (64, 1000, 1), (2, 21, 35), (1, 3, 1000)])
@pytest.mark.parametrize("use_log", [False, True])
def test_softmax_f32(ctx, orc, shape, use_log):
    outer, classes, inner = shape
    rng = np.random.Generator(np.random.PCG64(classes))
    x = (rng.standard_normal(shape) * 4).astype(np.float32)
    if shape == (2, 4, 1):
        x = np.array([1, 1, 1, 1, 1, 2, 3, 4], np.float32).reshape(shape)  # softmax_test.cc:37-38
    dx, do = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.softmax_f32(dx, do, outer, classes, inner, use_log)
    got = ctx.download(do, shape, np.float32)
    ref = orc.softmax_f32(x, outer, classes, inner, use_log).reshape(shape)
    # the reference's own softmax tests compare at 1e-5 (softmax_test.cc:96); expf on the
    # device and std::exp on the host differ by a few ulps
    assert np.abs(got - ref).max() <= (1e-4 if use_log else 1e-5)
    dx.free(); do.free()


@pytest.mark.parametrize("case", [
    # N, C, H, W, O, KH, stride, activation
    (3, 64, 16, 16, 160, 1, 1, 1),     # 1x1 stride 1, 256 pixels: sum + ReLU in the GEMM's epilogue, ragged N tile
    (2, 32, 12, 11, 48, 1, 1, 6),      # 132 pixels (a multiple of 4), LEAKYRELU
    (4, 40, 7, 7, 72, 1, 1, 1),        # 49 pixels: images merged, then one in-place sum + ReLU pass
    (2, 16, 14, 14, 24, 3, 1, 2),      # 3x3: convolution, then the in-place pass
    (1, 8, 9, 9, 8, 1, 2, 0),          # tiny: direct kernel, then the in-place pass
])
def test_conv2d_f32_residual(ctx, orc, case):
    """out = act((conv + bias) + residual) equals Conv2D (no activation), Eltwise SUM and
    Activation run one after the other."""
    N, C, H, W, O, k, st, act = case
    x, f, bias = _conv_inputs((N, C, H, W), (O, C, k, k), H * 7 + O)
    x = x * 2 - 1
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, k, k, (1, 1), (st, st), PAD["SAME"])
    rng = np.random.Generator(np.random.PCG64(O))
    res = rng.standard_normal((N, O, Ho, Wo)).astype(np.float32)
    conv = orc.conv2d_f32(x, f, bias, (st, st), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), 0)
    ref = orc.activation_f32(orc.eltwise_f32(conv, res, 0), act, 0.5, 0.1)
    dx, df, db, dr, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.upload(res), ctx.alloc(ref.nbytes)
    ctx.conv2d_f32_residual(dx, df, db, dr, do, N, C, H, W, O, k, k, (st, st), (1, 1), (ph >> 1, pw >> 1),
                            (Ho, Wo), act, 0.5, 0.1)
    assert rel_err(ctx.download(do, ref.shape, np.float32), ref, 1e-4, "conv2d_f32_residual") <= 1e-4
    for b in (dx, df, db, dr, do):
        b.free()



def test_zz_report_measured_errors():
    """Prints the worst measured errors of this module's comparisons (pytest -s shows them):
    the element-wise ratio |got - ref| / (abs_err + rel_err * |ref|) and the range-normalised
    error."""
    for label, (ratio, rng_err) in sorted(WORST.items()):
        print("%-32s element-wise ratio %.4f   range-normalised %.3e" % (label, ratio, rng_err))
    assert all(r <= 1.0 for r, _ in WORST.values())
