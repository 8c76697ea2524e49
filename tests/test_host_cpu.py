"""Host-side logic that needs no GPU: the delegator registry's error path, the configuration
class and logging (a small C++ program compiled here), batch sharding of the multi-GPU runner,
allocator fault injection, and the post-training-quantization range tooling."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_unit(tmp_path):
    """tests/host_unit.cc: an unknown delegator key gives MACE_UNSUPPORTED (the reference aborts,
    mace/core/registry/op_delegator_registry.cc:64-102), ConvType numbering, the MaceEngineConfig
    setters of include/mace/public/mace.h:372-499, LOG / VLOG / MACE_LATENCY_LOGGER."""
    exe = str(tmp_path / "host_unit")
    subprocess.check_call(["g++", "-std=c++17", "-O0", "-o", exe, os.path.join(ROOT, "tests", "host_unit.cc")])
    env = dict(os.environ)
    env.pop("MACE_CPP_MIN_VLOG_LEVEL", None)
    env.pop("MACE_CPP_MIN_LOG_LEVEL", None)
    out = subprocess.run([exe], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


def test_vlog_level_comes_from_the_environment():
    """MACE_CPP_MIN_VLOG_LEVEL / MACE_CPP_MIN_LOG_LEVEL are read once per process
    (include/mace/port/logger.h:40-58): ask a fresh process."""
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from mace_b200 import hostapi as H\n"
            "L = H.lib()\n"
            "print(L.mbh_vlog_is_on(0), L.mbh_vlog_is_on(2), L.mbh_vlog_is_on(3))\n" % ROOT)
    for env_extra, want in (({}, "1 0 0"), ({"MACE_CPP_MIN_VLOG_LEVEL": "2"}, "1 1 0"),
                            ({"MACE_CPP_MIN_VLOG_LEVEL": "3", "MACE_CPP_MIN_LOG_LEVEL": "W"}, "0 0 0")):
        env = {k: v for k, v in os.environ.items() if not k.startswith("MACE_CPP_")}
        env.update(env_extra)
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
        assert out.stdout.strip() == want, (env_extra, out.stdout, out.stderr)


def test_log_sink_and_levels():
    from mace_b200 import hostapi as H
    with H.LogCapture(vlog_level=1) as cap:
        H.lib().mbh_log(2, b"careful")
        assert H.lib().mbh_vlog_is_on(1) == 1 and H.lib().mbh_vlog_is_on(2) == 0
        assert H.lib().mbh_log(7, b"bad severity") == 1
    assert len(cap.lines) == 1 and cap.lines[0][0] == 2 and cap.lines[0][1].endswith("] careful")
    assert cap.lines[0][1].startswith("W ")


def test_shard_bounds_of_the_runner_match_the_process_level_rule():
    """The C++ MultiGpuRunner and the one-process-per-GPU helper split a batch the same way."""
    from mace_b200 import hostapi as H
    from mace_b200.sharding import shard_bounds
    for total in (0, 1, 2, 7, 64, 65, 256):
        for parts in (1, 2, 3, 4, 8):
            spans = [H.shard_bounds(total, parts, r) for r in range(parts)]
            assert spans == [shard_bounds(total, parts, r) for r in range(parts)]
            assert spans[0][0] == 0 and spans[-1][1] == total
    with pytest.raises(Exception):
        H.shard_bounds(4, 2, 2)


def test_runtime_failure_ratio_switch():
    """ShouldMockRuntimeFailure (mace/core/runtime_failure_mock.cc:25-53): never at ratio 0, always
    at 1, about the ratio in between; the ratio comes from MACE_RUNTIME_FAILURE_RATIO in a fresh
    process."""
    import mace_b200
    L = mace_b200.lib()
    try:
        assert L.mb_set_runtime_failure_ratio(0.0) == 0
        assert sum(L.mb_should_mock_runtime_failure() for _ in range(2000)) == 0
        assert L.mb_set_runtime_failure_ratio(1.0) == 0
        assert sum(L.mb_should_mock_runtime_failure() for _ in range(2000)) == 2000
        assert L.mb_set_runtime_failure_ratio(0.25) == 0
        hits = sum(L.mb_should_mock_runtime_failure() for _ in range(20000))
        assert 0.22 * 20000 < hits < 0.28 * 20000, hits
        assert L.mb_set_runtime_failure_ratio(1.5) == 1 and L.mb_set_runtime_failure_ratio(-0.1) == 1
    finally:
        L.mb_set_runtime_failure_ratio(0.0)
    code = ("import sys; sys.path.insert(0, %r)\n"
            "import mace_b200\n"
            "L = mace_b200.lib()\n"
            "print(sum(L.mb_should_mock_runtime_failure() for _ in range(1000)))\n" % ROOT)
    for value, lo, hi in ((None, 0, 0), ("1.0", 1000, 1000), ("0.5", 400, 600), ("junk", 0, 0)):
        env = {k: v for k, v in os.environ.items() if k != "MACE_RUNTIME_FAILURE_RATIO"}
        if value is not None:
            env["MACE_RUNTIME_FAILURE_RATIO"] = value
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
        assert lo <= int(out.stdout.strip()) <= hi, (value, out.stdout, out.stderr)


def test_quantize_stat_ranges_and_adjust_range(orc):
    """Range log -> per-tensor range (tools/python/quantize/quantize_stat.py:27-95) -> scale and
    zero point (quantize_util.py:102-122, the same numbers as the C++ AdjustRange)."""
    from mace_b200.harness import quantize_stat as qs
    rng = np.random.Generator(np.random.PCG64(3))
    log = ["I ops.cc:1] something else"]
    for run in range(20):
        log.append("I ops.cc:1300] Tensor range @@conv1@@%g,%g" % (-1.0 - 0.01 * run, 2.0 + 0.02 * run))
        log.append("I ops.cc:1300] Tensor range @@relu@@%g,%g" % (0.0, 6.0 if run != 7 else 60.0))
    got = dict(qs.overall_ranges(log))
    assert list(got) == ["conv1", "relu"]
    assert got["conv1"] == pytest.approx((-1.19, 2.38))
    assert got["relu"] == pytest.approx((0.0, 60.0))
    # a percentile trims the extremes of the per-run values
    assert dict(qs.overall_ranges(log, percentile=10))["relu"][1] == pytest.approx(6.0)
    # enhance mode gives up the one outlier run of "relu": the range shrinks by 90 % for 5 % of the runs
    assert dict(qs.overall_ranges(log, enhance=True, enhance_ratio=10))["relu"] == pytest.approx((0.0, 6.0))
    with pytest.raises(ValueError):
        qs.overall_ranges(["Tensor range @@t@@1.0,1.0"])
    for _ in range(200):
        lo, hi = sorted(rng.normal(0, 3, size=2).tolist())
        if hi - lo < 1e-3:
            continue
        for non_zero in (False, True):
            scale, zp, _, _ = qs.adjust_range(lo, hi, non_zero)
            s2, z2 = orc.adjust_range(np.float32(lo), np.float32(hi), non_zero)
            assert zp == z2 and scale == pytest.approx(float(s2), rel=1e-5)
