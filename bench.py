#!/usr/bin/env python
"""Benchmark of the uint8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (``config.workload``):
  gemm_u8_4096   uint8 MatMul M = N = K = 4096 (the compute-bound entry of the
                 K = N = 4096 sweep), zero points 128 / 120, fixed-point requantization
                 to uint8.  metric: u8 GEMM TOPS.

One "step" is one pass of the hot path over one batch of synthetic, seeded input.
`value` is measured with the inputs resident in HBM, `e2e` through the C ABI with
pinned HOST buffers (H2D + kernel + D2H inside the timed region).  Timing uses CUDA
events on the library's stream; with N > 1 each rank runs its own replica/shard, and
the time is the maximum over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML in a thread while the timed
    region runs (nvidia-smi reads the same counters, but takes longer to start than a short
    timed region lasts)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.masks = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.err = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # no NVML: report that instead of numbers
            self.err = "nvml unavailable: %s" % e
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.masks.add(int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)))
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(0.002)

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [self.err or "no samples"]}
        reasons = set()
        for m in self.masks:
            for bit, name in self.REASONS.items():
                if m & bit:
                    reasons.add(name)
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------
# workload: uint8 GEMM
# --------------------------------------------------------------------------------------

class GemmWorkload:
    name = "gemm_u8_4096"
    metric = "u8_gemm_tops"
    unit = "TOPS"
    dtype = "u8"

    def __init__(self, M=4096, N=4096, K=4096):
        self.M, self.N, self.K = M, N, K
        self.zp_a, self.zp_b = 128, 120
        self.ops_per_step = 2.0 * M * N * K
        # algorithmic bytes of one launch: A + B + C in uint8
        self.bytes_per_step = M * K + K * N + M * N

    def quant(self, orc):
        # output scale from the expected accumulator spread (std of a sum of K products of
        # centred uniform bytes), as AdjustRange would give for a +-4 sigma range
        sigma = np.sqrt(self.K) * 74.0 * 74.0
        s_c = np.float32(0.02 * 0.005 * 8 * sigma / 255.0)
        return orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.005), s_c) + (128,)

    def host_inputs(self, seed):
        rng = np.random.Generator(np.random.PCG64(seed))
        A = rng.integers(0, 256, size=(self.M, self.K), dtype=np.uint8)
        B = rng.integers(0, 256, size=(self.K, self.N), dtype=np.uint8)
        return A, B

    def config(self, n_sets):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K,
                "layout": "A row-major, B row-major (MN-major to the tensor core), C row-major",
                "zero_points": [self.zp_a, self.zp_b], "requant": "fixed-point -> uint8",
                "l2": "rotating %d operand sets (%.0f MB > L2)" % (
                    n_sets, n_sets * self.bytes_per_step / 1e6)}


def run_ours(args, rank, world):
    import mace_b200
    from oracle import pyoracle as orc  # only for quantization parameters and cpu_baseline
    local = int(os.environ.get("LOCAL_RANK", rank))
    ctx = mace_b200.Context(local)
    wl = GemmWorkload()
    mult, shift, zp_c = wl.quant(orc)
    n_sets = max(2, int(np.ceil(1.5 * L2_BYTES / wl.bytes_per_step)))
    sets = []
    for i in range(n_sets):
        A, B = wl.host_inputs(1000 * rank + i)
        sets.append((ctx.upload(A), ctx.upload(B), ctx.alloc(wl.M * wl.N)))

    def step(i):
        dA, dB, dC = sets[i % n_sets]
        ctx.gemm_u8(dA, dB, None, dC, 1, wl.M, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.01)
    l0, ltc0 = ctx.launches, ctx.launches_tensor_core
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for i in range(args.steps):
        step(i)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1)
    barrier()
    launches, launches_tc = ctx.launches - l0, ctx.launches_tensor_core - ltc0

    clocks = sampler.stop() if rank == 0 else None
    if args.profile:
        ctx.close()
        return None

    # end to end with host buffers: pinned H2D of A and B, GEMM, D2H of C, every step
    hA = ctx.host_alloc(wl.M * wl.K)
    hB = ctx.host_alloc(wl.K * wl.N)
    hC = ctx.host_alloc(wl.M * wl.N)
    A, B = wl.host_inputs(7)
    hA[:] = A.ravel()
    hB[:] = B.ravel()
    dA, dB, dC = sets[0]

    def e2e_step():
        ctx.h2d(dA, hA)
        ctx.h2d(dB, hB)
        ctx.gemm_u8(dA, dB, None, dC, 1, wl.M, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
        ctx.d2h(hC, dC)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 20))
    ctx.record(e0)
    for _ in range(e2e_steps):
        e2e_step()
    ctx.record(e1)
    e2e_ms = ctx.elapsed_ms(e0, e1)
    barrier()

    if dist is not None:
        import torch
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        value = world * wl.ops_per_step / (ms_per_step * 1e-3) / 1e12
        e2e_val = world * wl.ops_per_step / (e2e_ms / e2e_steps * 1e-3) / 1e12
        # int8 dense peak is not in MEASURED_PEAKS.json; the tensor core's int8 rate is twice
        # its bf16 rate, so the denominator is 2 x the measured bf16 burst figure.
        peak = 2.0 * peaks["bf16_tflops"]
        achieved = wl.ops_per_step / (ms_per_step * 1e-3) / 1e12
        result = {
            "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(n_sets), parallelism="replicas only (dp%d)" % world),
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2),
                         "peak": round(peak, 1), "unit": "TOP/s",
                         "frac": round(achieved / peak, 4), "traffic": None,
                         "peak_source": "2 x %s bf16 burst (int8 rate of the tensor core)"
                                        % peaks["source"],
                         "kernel": "gemm_u8_tc_kernel<256> + operand byte-sum kernels"},
            "e2e": {"value": round(e2e_val, 3), "unit": wl.unit,
                    "h2d_bytes_per_step": wl.M * wl.K + wl.K * wl.N,
                    "d2h_bytes_per_step": wl.M * wl.N},
            "gpu_launches": launches, "gpu_launches_tensor_core": launches_tc,
            "clocks": clocks,
        }
        result["cpu_baseline"] = cpu_baseline(wl, orc, mult, shift, zp_c, steps=2)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return result


def cpu_baseline(wl, orc, mult, shift, zp_c, steps):
    """The oracle (a port of the reference's CPU arithmetic) on this box's host cores."""
    A, B = wl.host_inputs(0)
    # bounded sample: the first 1024 rows of A against the whole B
    rows = min(wl.M, 1024)
    threads = orc.set_threads(0)
    orc.gemm_u8(A[:64], B, None, 1, 64, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.gemm_u8(A[:rows], B, None, 1, rows, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    dt = (time.perf_counter() - t0) / steps
    return {"value": round(2.0 * rows * wl.N * wl.K / dt / 1e12, 5), "unit": wl.unit,
            "cores": threads, "kind": "port",
            "sample": "%d of %d rows of A against all of B, %d passes" % (rows, wl.M, steps)}


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path: the oracle port (the reference's own
    sources need NEON, gemmlowp and protobuf, none of which exist here)."""
    if rank != 0:
        return None
    from oracle import pyoracle as orc
    wl = GemmWorkload()
    mult, shift, zp_c = wl.quant(orc)
    A, B = wl.host_inputs(0)
    rows = min(wl.M, 1024)
    threads = orc.set_threads(0)
    for _ in range(min(args.warmup, 1) or 1):
        orc.gemm_u8(A[:64], B, None, 1, 64, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.gemm_u8(A[:rows], B, None, 1, rows, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    dt = (time.perf_counter() - t0) / steps
    value = round(2.0 * rows * wl.N * wl.K / dt / 1e12, 5)
    sample = "%d of %d rows of A against all of B per step" % (rows, wl.M)
    return {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit,
            "n_gpus": world, "steps": steps, "warmup": 1,
            "ms_per_step": round(dt * 1e3 * wl.M / rows, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(1), parallelism="host cores"),
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile", action="store_true",
                    help="run only the device-resident timed loop (for ncu captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        res = run_reference(args, rank, world)
    else:
        res = run_ours(args, rank, world)
    if rank == 0 and res is not None:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
