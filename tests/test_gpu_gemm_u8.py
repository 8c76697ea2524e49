"""uint8 GEMM on the GPU against the CPU oracle: bit-exact."""
import numpy as np
import pytest

from helpers import gemm_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import mace_b200
    c = mace_b200.Context(0)
    yield c
    c.close()


def run_gemm(ctx, orc, case, batch, M, N, K, out_int32=False, c_col_major=False,
             bias_per_row=False, **kw):
    A, B, bias = ctx.upload(case["A"]), ctx.upload(case["B"]), None
    if case["bias"] is not None:
        bias = ctx.upload(case["bias"])
    itemsize = 4 if out_int32 else 1
    out = ctx.alloc(batch * M * N * itemsize + 64)
    # canary bytes after the output
    ctx._check(__import__("mace_b200").lib().mb_memset(ctx.h, out.ptr, 0xA5, out.nbytes))
    ctx.gemm_u8(A, B, bias, out, batch, M, N, K, case["zp_a"], case["zp_b"], case["mult"],
                case["shift"], case["zp_c"], c_col_major=c_col_major, out_int32=out_int32,
                bias_per_row=bias_per_row, **kw)
    got_all = ctx.download(out, (out.nbytes,), np.uint8)
    assert (got_all[batch * M * N * itemsize:] == 0xA5).all(), "wrote past the output"
    got = got_all[:batch * M * N * itemsize].view(np.int32 if out_int32 else np.uint8)
    exp = orc.gemm_u8(case["A"], case["B"], case["bias"], batch, M, N, K, case["zp_a"],
                      case["zp_b"], case["mult"], case["shift"], case["zp_c"],
                      c_col_major=c_col_major, out_int32=out_int32, bias_per_row=bias_per_row,
                      **kw)
    for b in (A, B, out):
        b.free()
    return got, exp


def test_config0_1024_matmul(ctx, orc):
    """M=N=K=1024, zero points 128/120, scales 0.02/0.005, seed 0 (MatMul: no bias)."""
    case = gemm_case(orc, 0, 1, 1024, 1024, 1024)
    before = ctx.launches_tensor_core
    got, exp = run_gemm(ctx, orc, case, 1, 1024, 1024, 1024)
    assert ctx.launches_tensor_core == before + 1, "tensor-core kernel did not run"
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 100  # a vacuous all-saturated output would prove nothing


def test_config0_1024_with_bias_conv_form(ctx, orc):
    """The biased GEMM of the same config: bias per output channel (Conv2D 1x1 form)."""
    case = gemm_case(orc, 0, 1, 1024, 1024, 1024, bias_len=1024)
    got, exp = run_gemm(ctx, orc, case, 1, 1024, 1024, 1024, bias_per_row=True)
    assert np.array_equal(got, exp)
    got, exp = run_gemm(ctx, orc, case, 1, 1024, 1024, 1024, bias_per_row=False)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("a_cm,b_cm", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mn_major", [1, 0])
def test_transpose_combos_tensor_core(ctx, orc, a_cm, b_cm, mn_major):
    """All four transpose_a/transpose_b combinations (matmul_test.cc:162-254), aligned so
    that the tensor-core path takes them, with MN-major operands either described to the
    tensor core directly or transposed in scratch."""
    ctx.set_option("mn_major", mn_major)
    try:
        M, N, K = 256, 384, 512
        case = gemm_case(orc, 3, 1, M, N, K, a_col_major=a_cm, b_col_major=b_cm)
        before = ctx.launches_tensor_core
        got, exp = run_gemm(ctx, orc, case, 1, M, N, K, a_col_major=a_cm, b_col_major=b_cm)
        assert ctx.launches_tensor_core == before + 1
        assert np.array_equal(got, exp)
    finally:
        ctx.set_option("mn_major", 1)


@pytest.mark.parametrize("shape", [(1, 31, 61, 67), (2, 16, 32, 48), (3, 128, 64, 16),
                                   (1, 1, 256, 30000 // 16 * 16), (1, 200, 136, 144),
                                   (16, 64, 64, 64), (1, 129, 272, 4096)])
def test_shapes_and_tails(ctx, orc, shape):
    batch, M, N, K = shape
    case = gemm_case(orc, 11, batch, M, N, K)
    got, exp = run_gemm(ctx, orc, case, batch, M, N, K)
    assert np.array_equal(got, exp)


def test_config4_m128_and_batched_512(ctx, orc):
    """The two sweep shapes that sit between the few-row kernel and the square GEMM: M = 128
    against K = N = 4096 (one row of 128-row tiles), and the batched 64 x 512^3 MatMul.  Every
    output byte against the oracle, with and without a bias; for the batched product each of
    four sampled entries is also run alone (one batch entry) and must give the same bytes as
    it does inside the batch."""
    M, N, K = 128, 4096, 4096
    for bias_len in (None, N):
        case = gemm_case(orc, 41, 1, M, N, K, bias_len=bias_len)
        before = ctx.launches_tensor_core
        got, exp = run_gemm(ctx, orc, case, 1, M, N, K)
        assert ctx.launches_tensor_core > before, "tensor-core kernel did not run"
        assert np.array_equal(got, exp)
        assert len(np.unique(got)) > 100
    batch, M, N, K = 64, 512, 512, 512
    case = gemm_case(orc, 42, batch, M, N, K)
    got, exp = run_gemm(ctx, orc, case, batch, M, N, K)
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 100
    got = got.reshape(batch, M, N)
    for b in (0, 17, 40, 63):
        one = dict(case, A=np.ascontiguousarray(case["A"][b:b + 1]), B=np.ascontiguousarray(case["B"][b:b + 1]))
        alone, exp1 = run_gemm(ctx, orc, one, 1, M, N, K)
        assert np.array_equal(alone, exp1)
        assert np.array_equal(alone.reshape(M, N), got[b])


@pytest.mark.parametrize("a_cm,b_cm", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 1024, 4096), (16, 2048, 2048), (100, 512, 3072), (200, 640, 2048)])
def test_depth_cut_into_runs(ctx, orc, shape, a_cm, b_cm):
    """Few output tiles and a long depth: the product runs as several depth runs over more SMs
    plus a kernel that adds the int32 partial results (operand sums per run for MN-major
    operands, inside the kernel for K-major ones).  Every byte against the oracle and against
    the undivided product: zero points on either side or none, bias per column / per row /
    none, uint8 and int32 output."""
    M, N, K = shape
    if a_cm and M % 16 != 0:
        pytest.skip("MN-major A with M % 16 != 0 goes through a K-major copy, which is not cut")
    variants = [dict(zp_a=128, zp_b=120, bias_len=N), dict(zp_a=0, zp_b=0), dict(zp_a=7, zp_b=0, bias_len=M),
                dict(zp_a=0, zp_b=255)]
    for i, v in enumerate(variants):
        per_row = v.get("bias_len") == M and M != N
        case = gemm_case(orc, 50 + i, 1, M, N, K, bias_len=v.get("bias_len"), a_col_major=a_cm, b_col_major=b_cm,
                         zp_a=v["zp_a"], zp_b=v["zp_b"])
        for out_int32 in ((False, True) if i < 2 else (False,)):
            got = {}
            for split in (1, 0):
                ctx.set_option("split_k", split)
                ctx.set_option("skinny_max_m", 0)
                try:
                    before = ctx.launches
                    got[split], exp = run_gemm(ctx, orc, case, 1, M, N, K, a_col_major=a_cm, b_col_major=b_cm,
                                               out_int32=out_int32, bias_per_row=per_row)
                    launches = ctx.launches - before
                finally:
                    ctx.set_option("split_k", 1)
                    ctx.set_option("skinny_max_m", 16)
                assert np.array_equal(got[split], exp), (split, v, out_int32)
                if split:
                    assert launches in (2, 3), launches  # [operand sums,] the runs, the add-up kernel
                else:
                    assert launches in (1, 2), launches
            if not out_int32 and i == 0:
                assert len(np.unique(got[1])) > 50


@pytest.mark.parametrize("a_cm,b_cm", [(False, False), (False, True), (True, False), (True, True)])
def test_unaligned_generic_path(ctx, orc, a_cm, b_cm):
    """31 x 61 x 67 (matmul_test.cc): no 16-byte alignment anywhere, CUDA-core kernel."""
    case = gemm_case(orc, 5, 2, 31, 67, 61, a_col_major=a_cm, b_col_major=b_cm)
    before = ctx.launches_tensor_core
    got, exp = run_gemm(ctx, orc, case, 2, 31, 67, 61, a_col_major=a_cm, b_col_major=b_cm)
    assert ctx.launches_tensor_core == before
    assert np.array_equal(got, exp)


def test_one_side_batched_and_int32_and_colmajor_out(ctx, orc):
    M, N, K = 96, 160, 208
    case = gemm_case(orc, 7, 3, M, N, K, b_batched=False)
    got, exp = run_gemm(ctx, orc, case, 3, M, N, K, b_batched=False)
    assert np.array_equal(got, exp)
    case = gemm_case(orc, 8, 3, M, N, K, a_batched=False)
    got, exp = run_gemm(ctx, orc, case, 3, M, N, K, a_batched=False, out_int32=True)
    assert np.array_equal(got, exp)
    case = gemm_case(orc, 9, 1, M, N, K, bias_len=M)
    got, exp = run_gemm(ctx, orc, case, 1, M, N, K, c_col_major=True, bias_per_row=True)
    assert np.array_equal(got, exp)
    got, exp = run_gemm(ctx, orc, case, 1, M, N, K, c_col_major=True, out_int32=True,
                        bias_per_row=True)
    assert np.array_equal(got, exp)


def test_tensor_core_matches_cuda_core_kernel(ctx, orc):
    M, N, K = 384, 512, 1024
    case = gemm_case(orc, 21, 1, M, N, K, bias_len=N)
    got_tc, exp = run_gemm(ctx, orc, case, 1, M, N, K)
    ctx.set_option("tensor_cores", 0)
    try:
        before = ctx.launches_tensor_core
        got_cc, _ = run_gemm(ctx, orc, case, 1, M, N, K)
        assert ctx.launches_tensor_core == before
    finally:
        ctx.set_option("tensor_cores", 1)
    assert np.array_equal(got_tc, exp) and np.array_equal(got_cc, exp)


def test_extreme_zero_points_and_saturation(ctx, orc):
    M, N, K = 128, 128, 256
    for zp_a, zp_b in [(0, 0), (255, 255), (0, 255), (1, 0)]:
        case = gemm_case(orc, 13, 1, M, N, K, zp_a=zp_a, zp_b=zp_b)
        got, exp = run_gemm(ctx, orc, case, 1, M, N, K)
        assert np.array_equal(got, exp)
    # all-zero and all-255 operands
    case = gemm_case(orc, 13, 1, M, N, K)
    case["A"][:] = 255
    case["B"][:] = 255
    got, exp = run_gemm(ctx, orc, case, 1, M, N, K, out_int32=True)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("zp_c", [0, 255, 100])
@pytest.mark.parametrize("shift", [0, 1, 9, 31])
def test_requantization_variants(ctx, orc, zp_c, shift):
    """Every epilogue variant (output zero point 0 or not, shift 0 or not) with
    accumulators of both signs, ties of the rounding shift and int32 biases near the
    limits of the range."""
    M, N, K = 128, 96, 64
    case = gemm_case(orc, 11 + shift, 1, M, N, K, bias_len=N)
    case["zp_c"], case["shift"] = zp_c, shift
    case["mult"] = 1518500250 if shift else 1 << 30
    bias = case["bias"].astype(np.int64)
    bias[::7] = 2 ** 31 - 1 - 255 * 255 * K
    bias[3::7] = -2 ** 31 + 255 * 255 * K
    if shift >= 1:  # exact ties of the second rounding stage around zero
        bias[1::5] = (1 << shift) >> 1
        bias[2::5] = -((1 << shift) >> 1)
    case["bias"] = bias.astype(np.int32)
    if shift <= 1:  # keep some accumulators small enough not to saturate
        case["A"][:, ::2, :] = case["zp_a"]
        case["A"][:, ::2, :3] += np.arange(3, dtype=np.uint8)
    got, exp = run_gemm(ctx, orc, case, 1, M, N, K)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 4096, 4096), (3, 640, 260), (7, 516, 1000),
                                   (9, 2048, 512)])
@pytest.mark.parametrize("out_int32", [False, True])
def test_few_rows_against_row_major_b(ctx, orc, shape, out_int32):
    """M <= 16 with a row-major B (the M = 1 / M = 16 cases of the K = N = 4096 sweep): the
    CUDA-core streaming kernel, twice in a row (its workspace must come back zeroed), with a
    bias, ragged N and K, and interleaved with a differently shaped call.  (With the default
    options M = 16 against 4096 x 4096 goes to the tensor core over depth runs instead, which
    test_depth_cut_into_runs covers; here that route is switched off.)"""
    M, N, K = shape
    case = gemm_case(orc, M + N, 1, M, N, K, bias_len=N)
    if M >= 2 and K >= 2048:
        before = ctx.launches_tensor_core
        got, exp = run_gemm(ctx, orc, case, 1, M, N, K, out_int32=out_int32)
        assert np.array_equal(got, exp)
        assert ctx.launches_tensor_core > before, "expected the tensor-core kernel over depth runs"
    ctx.set_option("split_k", 0)
    try:
        before = ctx.launches_tensor_core
        for _ in range(2):
            got, exp = run_gemm(ctx, orc, case, 1, M, N, K, out_int32=out_int32)
            assert np.array_equal(got, exp)
        assert ctx.launches_tensor_core == before, "expected the CUDA-core streaming kernel"
    finally:
        ctx.set_option("split_k", 1)
    other = gemm_case(orc, 5, 1, 2, 512, 256, bias_len=2)
    got, exp = run_gemm(ctx, orc, other, 1, 2, 512, 256, bias_per_row=True)
    assert np.array_equal(got, exp)
    got, exp = run_gemm(ctx, orc, case, 1, M, N, K, out_int32=out_int32)
    assert np.array_equal(got, exp)
    if not out_int32:
        assert len(np.unique(got)) > 16


@pytest.mark.parametrize("shape", [(256, 256, 512, False, False, 1), (384, 320, 640, False, False, 1),
                                   (512, 256, 256, True, False, 1), (272, 528, 384, True, True, 2),
                                   (640, 1024, 2048, False, True, 1)])
def test_cta_pair_kernel(ctx, orc, shape):
    """The GEMM on clusters of two CTAs (one 256 x 256 tile per pair, the even CTA issuing the
    MMAs for both, each CTA loading its half of the operands and draining its own 128 rows):
    all four operand orders, ragged M and N (the odd CTA's rows partly or wholly outside the
    matrix), a batch, several tiles per pair; every byte against the oracle and against the
    one-CTA kernel."""
    M, N, K, a_cm, b_cm, batch = shape
    case = gemm_case(orc, 7, batch, M, N, K, bias_len=N, a_col_major=a_cm, b_col_major=b_cm)
    got = {}
    for pair in (2, 0):
        ctx.set_option("pair", pair)
        ctx.set_option("split_k", 0)
        try:
            before = ctx.launches_pair
            got[pair], exp = run_gemm(ctx, orc, case, batch, M, N, K, a_col_major=a_cm, b_col_major=b_cm)
            assert (ctx.launches_pair - before) == (1 if pair else 0)
        finally:
            ctx.set_option("pair", 0)
            ctx.set_option("split_k", 1)
        assert np.array_equal(got[pair], exp), pair
    assert len(np.unique(got[2])) > 50


@pytest.mark.parametrize("force_bn", [0, 64, 128, 256])
@pytest.mark.parametrize("shape", [(200, 272, 1000), (128, 256, 1024), (77, 112, 48), (300, 528, 144)])
def test_column_sums_from_row_major_b_tiles(ctx, orc, shape, force_bn):
    """K-major A against a row-major B with a depth of at most 1024: no sums kernel runs, the
    preparation warps add B's columns from the swizzled tiles (16-bit count pairs per 32 depth
    rows, the four warps' quarters joined in shared memory).  Ragged M, N and K (a last K block
    that TMA fills with zeros), every tile width, all-255 operands (no count may wrap), either
    zero point alone; every byte against the oracle."""
    M, N, K = shape
    rng = np.random.Generator(np.random.PCG64(M + N + K))
    if force_bn:
        ctx.set_option("force_bn", force_bn)
    try:
        for zp_a, zp_b, fill in ((128, 120, None), (255, 0, None), (0, 255, None), (128, 120, 255)):
            A = rng.integers(0, 256, size=(1, M, K), dtype=np.uint8)
            B = rng.integers(0, 256, size=(1, K, N), dtype=np.uint8)
            if fill is not None:
                A[:] = fill
                B[:] = fill
            bias = np.rint(rng.normal(0, 1000, size=N)).astype(np.int32)
            acc = orc.gemm_u8(A, B, None, 1, M, N, K, zp_a, zp_b, out_int32=True).astype(np.float64)
            s_c = max(float(np.abs(acc).max()), 1.0) * 1e-4 / 127.0
            mult, shift = orc.output_multiplier_and_shift(np.float32(0.01), np.float32(0.01), np.float32(s_c))
            case = dict(A=A, B=B, bias=bias, zp_a=zp_a, zp_b=zp_b, mult=mult, shift=shift, zp_c=128)
            before = ctx.launches
            got, exp = run_gemm(ctx, orc, case, 1, M, N, K)
            assert ctx.launches - before == 1, "expected the GEMM alone (sums from its tiles)"
            assert np.array_equal(got, exp), (zp_a, zp_b, fill)
    finally:
        ctx.set_option("force_bn", 0)


def test_empty_and_bad_arguments(ctx):
    import mace_b200
    buf = ctx.alloc(64)
    # empty output: success, nothing written
    ctx.gemm_u8(buf, buf, None, buf, 0, 4, 4, 4, 0, 0)
    ctx.gemm_u8(buf, buf, None, buf, 1, 0, 4, 4, 0, 0)
    with pytest.raises(mace_b200.MaceB200Error) as e:
        ctx.gemm_u8(buf, buf, None, buf, 1, -1, 4, 4, 0, 0)
    assert e.value.code == 1
    with pytest.raises(mace_b200.MaceB200Error) as e:
        ctx.gemm_u8(buf, buf, None, buf, 1, 4, 4, 4, 0, 0, mult=0)
    assert e.value.code == 1
    with pytest.raises(mace_b200.MaceB200Error) as e:
        ctx.gemm_u8(buf, buf, None, buf, 1, 4, 4, 4, 0, 0, shift=40)
    assert e.value.code == 1


def test_linearity_at_full_size(ctx, orc):
    """K = N = 4096, M = 4096 is too large for the scalar oracle in seconds; check raw int32
    accumulators through properties instead: (a) a random sample of rows against the oracle,
    (b) additivity over a split of K."""
    M = N = K = 4096
    rng = np.random.Generator(np.random.PCG64(4))
    A = rng.integers(0, 256, size=(M, K), dtype=np.uint8)
    B = rng.integers(0, 256, size=(K, N), dtype=np.uint8)
    dA, dB = ctx.upload(A), ctx.upload(B)
    out = ctx.alloc(M * N * 4)
    ctx.gemm_u8(dA, dB, None, out, 1, M, N, K, 128, 120, out_int32=True)
    full = ctx.download(out, (M, N), np.int32)
    rows = rng.choice(M, size=16, replace=False)
    exp = orc.gemm_u8(A[rows], B, None, 1, 16, N, K, 128, 120, out_int32=True).reshape(16, N)
    assert np.array_equal(full[rows], exp)
    # additivity over K: C(K) = C(first half) + C(second half)
    A1, A2 = np.ascontiguousarray(A[:, :K // 2]), np.ascontiguousarray(A[:, K // 2:])
    B1, B2 = np.ascontiguousarray(B[:K // 2]), np.ascontiguousarray(B[K // 2:])
    parts = []
    for a, b in ((A1, B1), (A2, B2)):
        da, db = ctx.upload(a), ctx.upload(b)
        ctx.gemm_u8(da, db, None, out, 1, M, N, K // 2, 128, 120, out_int32=True)
        parts.append(ctx.download(out, (M, N), np.int32))
        da.free()
        db.free()
    assert np.array_equal(full, parts[0] + parts[1])
    # the requantized uint8 output of the same product (tensor-core kernel, TMA-store epilogue):
    # sampled rows against the oracle, and every output byte as a function of the int32 result
    case = gemm_case(orc, 0, 1, 64, 64, 64)  # only for plausible multiplier / shift / zero point
    mult, shift, zp_c = case["mult"], 9, 128
    out8 = ctx.alloc(M * N)
    before = ctx.launches_tensor_core
    ctx.gemm_u8(dA, dB, None, out8, 1, M, N, K, 128, 120, mult, shift, zp_c)
    assert ctx.launches_tensor_core == before + 1
    got8 = ctx.download(out8, (M, N), np.uint8)
    exp8 = orc.gemm_u8(A[rows], B, None, 1, 16, N, K, 128, 120, mult, shift, zp_c).reshape(16, N)
    assert np.array_equal(got8[rows], exp8)
    requant = np.array([min(255, max(0, orc.rounding_stages(int(v), mult, shift) + zp_c))
                        for v in np.unique(full)[::4001]], dtype=np.uint8)
    lut = dict(zip(np.unique(full)[::4001].tolist(), requant.tolist()))
    flat_full, flat8 = full.ravel(), got8.ravel()
    for v, q in list(lut.items())[:200]:
        assert (flat8[flat_full == v] == q).all()
    assert len(np.unique(got8)) > 100


@pytest.mark.parametrize("N,K", [(64, 32), (128, 64), (128, 128), (256, 256), (512, 512), (1024, 96)])
def test_pointwise_shapes_with_many_tiles_per_cta(ctx, orc, N, K):
    """Pointwise-convolution shapes ([pixels x K] * [N x K]^T, K-major operands) large enough
    that every persistent CTA walks through its accumulator buffers several times; sampled
    rows against the oracle, three runs (a race shows up as run-to-run differences)."""
    M = 148 * 128 * 3 + 77
    rng = np.random.Generator(np.random.PCG64(N + K))
    A = rng.integers(0, 256, size=(1, M, K), dtype=np.uint8)
    Bt = rng.integers(1, 256, size=(1, N, K), dtype=np.uint8)  # stored [N x K] = column-major B
    bias = np.rint(rng.normal(0, 2000, size=N)).astype(np.int32)
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01),
                                                  np.float32(0.02 * 0.01 * np.sqrt(K) * 74 * 74 * 3 / 127))
    dA, dB, db = ctx.upload(A), ctx.upload(Bt), ctx.upload(bias)
    out = ctx.alloc(M * N)
    rows = np.sort(rng.choice(M, size=48, replace=False))
    rows[-1] = M - 1
    exp = orc.gemm_u8(np.ascontiguousarray(A[:, rows]), Bt, bias, 1, len(rows), N, K, 0, 131, mult, shift, 0,
                      b_col_major=True).reshape(len(rows), N)
    first = None
    for _ in range(3):
        ctx.gemm_u8(dA, dB, db, out, 1, M, N, K, 0, 131, mult, shift, 0, b_col_major=True)
        got = ctx.download(out, (M, N), np.uint8)
        assert np.array_equal(got[rows], exp)
        if first is None:
            first = got
        else:
            assert np.array_equal(got, first)
    assert len(np.unique(first)) > 50
    for b in (dA, dB, db, out):
        b.free()
