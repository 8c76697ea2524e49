"""The allocation-free GEMM entry point, mb_gemm_u8_static_scratch.

Some callers of this library cannot call cudaMalloc at the moment they need a GEMM (a
real-time loop with a fixed memory budget, a plugin whose host application owns all device
memory, a callback that may run during a stream capture).  For them the library keeps the
GEMM's scratch -- the operand byte sums and the kernel's status word -- in a fixed array
that ships with the library.  This test calls that entry point through the C ABI twice in a
row, with different problem sizes so that anything left in the shared array by the first
call would corrupt the second, and requires the same bytes as mb_gemm_u8 produces and as the
CPU oracle computes; after each call it also reads the kernel's status word back through
mb_gemm_u8_static_scratch_status (a bounded wait that ran out would otherwise go unnoticed,
because this entry point has no context whose sync could report it).

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import gemm_case

pytestmark = pytest.mark.gpu


def _run_pair(ctx, lib, orc, seed, M, N, K, a_cm, b_cm, bias_per_row):
    case = gemm_case(orc, seed, 1, M, N, K, bias_len=(M if bias_per_row else N),
                     a_col_major=a_cm, b_col_major=b_cm)
    A, B, bias = ctx.upload(case["A"]), ctx.upload(case["B"]), ctx.upload(case["bias"])
    ref_out, new_out = ctx.alloc(M * N), ctx.alloc(M * N)
    ctx.gemm_u8(A, B, bias, ref_out, 1, M, N, K, case["zp_a"], case["zp_b"], case["mult"],
                case["shift"], case["zp_c"], a_col_major=a_cm, b_col_major=b_cm,
                bias_per_row=bias_per_row)
    expected = ctx.download(ref_out, (M, N), np.uint8)
    msg = C.create_string_buffer(256)
    st = lib.mb_gemm_u8_static_scratch(
        ctx.stream, A.ptr, B.ptr, bias.ptr, new_out.ptr, 0, M, N, K, int(a_cm), int(b_cm),
        case["zp_a"], case["zp_b"], case["mult"], case["shift"], case["zp_c"],
        int(bias_per_row), msg, len(msg))
    assert st == 0, msg.value.decode()
    status = C.c_int(-1)
    assert lib.mb_gemm_u8_static_scratch_status(ctx.stream, C.byref(status)) == 0
    got = ctx.download(new_out, (M, N), np.uint8)  # synchronizes the stream
    assert status.value == 0, "the kernel gave up a bounded wait (code %d)" % status.value
    # integer arithmetic: the tolerance of the uint8 tests is exact equality
    assert np.array_equal(got, expected)
    oracle = orc.gemm_u8(case["A"], case["B"], case["bias"], 1, M, N, K, case["zp_a"], case["zp_b"],
                         case["mult"], case["shift"], case["zp_c"], a_col_major=a_cm,
                         b_col_major=b_cm, bias_per_row=bias_per_row).reshape(M, N)
    assert np.array_equal(got, oracle)
    assert len(np.unique(got)) > 16
    for b in (A, B, bias, ref_out, new_out):
        b.free()


def test_static_scratch_gemm_matches_mb_gemm_u8_twice_in_a_row(orc):
    import mace_b200
    lib = mace_b200.lib()
    ctx = mace_b200.Context(0)
    try:
        # first call: the larger problem; second call: a smaller one with other layouts, so
        # stale sums from the first call would show
        _run_pair(ctx, lib, orc, 41, 640, 768, 512, False, False, False)
        _run_pair(ctx, lib, orc, 42, 256, 384, 1024, True, True, True)
    finally:
        ctx.close()


def test_static_scratch_gemm_rejects_what_it_cannot_hold():
    import mace_b200
    lib = mace_b200.lib()
    ctx = mace_b200.Context(0)
    try:
        buf = ctx.alloc(1 << 16)
        msg = C.create_string_buffer(256)
        too_big = 16384 + 16
        st = lib.mb_gemm_u8_static_scratch(ctx.stream, buf.ptr, buf.ptr, None, buf.ptr, 0,
                                           too_big, 16, 16, 0, 0, 0, 0, 1 << 30, 0, 0, 0, msg,
                                           len(msg))
        assert st == 1 and b"limit" in msg.value
        st = lib.mb_gemm_u8_static_scratch(ctx.stream, buf.ptr, buf.ptr, None, buf.ptr, 0,
                                           31, 67, 61, 0, 0, 0, 0, 1 << 30, 0, 0, 0, msg,
                                           len(msg))
        assert st == 3 and b"16" in msg.value
        # zero points outside uint8 are rejected before anything is enqueued
        st = lib.mb_gemm_u8_static_scratch(ctx.stream, buf.ptr, buf.ptr, None, buf.ptr, 0,
                                           64, 64, 64, 0, 0, 0, 0, 1 << 30, 0, 256, 0, msg,
                                           len(msg))
        assert st == 1 and b"zero point" in msg.value
        st = lib.mb_gemm_u8_static_scratch(ctx.stream, buf.ptr, buf.ptr, None, buf.ptr, 0,
                                           64, 64, 64, 0, 0, -1, 0, 1 << 30, 0, 0, 0, msg,
                                           len(msg))
        assert st == 1 and b"zero point" in msg.value
    finally:
        ctx.close()
