#!/usr/bin/env python
"""Benchmark of the uint8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (``config.workload``):
  mobilenet_v1_u8_b64  (default) quantized MobileNet-v1 1.0, 224x224, batch 64 per GPU, uint8
                 NHWC, random seeded weights, through the C++ host engine (operators ->
                 delegators -> C ABI).  metric: images/s.  The line also carries the u8 GEMM
                 TOPS of the 4096^3 MatMul under "u8_gemm".
  gemm_u8_4096   uint8 MatMul M = N = K = 4096, zero points 128 / 120, fixed-point
                 requantization to uint8.  metric: u8 GEMM TOPS.
  winograd_f32_cfg1  fp32 3x3 Conv2D, input [32,64,56,56], filter [64,64,3,3], SAME, through the
                 Winograd entry point (cached transformed filter).  metric: direct-equivalent TFLOP/s.
  gemm_u8_sweep  uint8 GEMM with K = N = 4096 and M in {1, 16, 128, 4096}, the batched
                 64 x 512^3 MatMul and the 4096 x 4096 GEMV; one row per case under "cases".
  resnet50_f32_b256  ResNet-50 v1, fp32 NCHW, 224x224, batch 256 per GPU (--batch changes it),
                 He-normal seeded weights, through the C++ host engine: 3x3 convolutions by
                 Winograd, 1x1 by GEMM, stem and stride-2 1x1 by im2col + GEMM, pooling, residual
                 sums and activations on the device.  metric: images/s.

One "step" is one pass of the hot path over one batch of synthetic, seeded input.  `value`
is measured with the inputs resident in HBM, `e2e` through the host-buffer entry point with
pinned HOST buffers (H2D + kernels + D2H inside the timed region).  Timing uses CUDA events on
the library's stream; with N > 1 each rank runs its own shard (weak scaling: the per-GPU batch
is fixed) and the time is the maximum over ranks; the logits are gathered every step by one
all_gather on a side stream, and "strong_scaling" repeats the measurement with the
configuration's own batch of 64 split over the ranks.

The default line also carries: "tensor_peaks_measured" (int8 and tf32 library GEMMs timed on
this GPU: the denominators of every tensor-bound fraction), "u8_gemm" (the 4096^3 MatMul),
"configs" (compact records of the other configurations: 1024^3, the Winograd convolution, the
K = N = 4096 sweep with the batched MatMul and the GEMV, ResNet-50 at batch 256; --no-extras
skips them), "kernel_families_ms", "h2d_gbs_per_rank", "e2e_model_api" and "cpu_baseline".
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum from the ncu captures summarised under profiles/
# (bytes per step of the kernel family, resp. per launch); outputs that are still in L2 when a
# kernel's capture ends are not in these sums.
NCU_TRAFFIC = {
    "mobilenet_dw": 196.8e6,   # 13 depthwise launches, profiles/mobilenet_v1_u8_b64_launches.md
    "mobilenet_pw": 130.3e6,   # 13 pointwise + FC GEMM launches, same file
    "gemm_u8_4096": 35.0e6,    # gemm_u8_tc_kernel<256>, profiles/gemm_u8_tc_kernel_4096.md
    "winograd_f32_cfg1": 134.6e6,  # three kernels of one convolution, caches flushed between them
}


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


def library_tensor_peaks(device_index, seconds=2.0):
    """int8 and tf32 tensor-core yardsticks measured on this GPU with library GEMMs, the way
    MEASURED_PEAKS.json's bf16 figure is made: 8192^3, best of 10 launches (burst) and back to
    back for `seconds` (sustained), CUDA events, SM clocks sampled meanwhile.  torch._int_mm is
    cuBLASLt's int8 x int8 -> int32 GEMM, torch.matmul with TF32 allowed its tf32 GEMM.  These
    are denominators only; nothing of the measured path calls them."""
    import torch
    out = {}
    dev = torch.device("cuda", device_index)
    n = 8192
    ops = 2.0 * n ** 3
    with torch.cuda.device(dev):
        a8 = torch.randint(-128, 127, (n, n), dtype=torch.int8, device=dev)
        b8 = torch.randint(-128, 127, (n, n), dtype=torch.int8, device=dev)
        a32 = torch.randn((n, n), dtype=torch.float32, device=dev)
        b32 = torch.randn((n, n), dtype=torch.float32, device=dev)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            for key, fn in (("int8", lambda: torch._int_mm(a8, b8)), ("tf32", lambda: torch.matmul(a32, b32))):
                try:
                    for _ in range(3):
                        fn()
                    torch.cuda.synchronize()
                    best = float("inf")
                    for _ in range(10):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        fn()
                        e1.record()
                        e1.synchronize()
                        best = min(best, e0.elapsed_time(e1))
                    sampler = ClockSampler(device_index)
                    sampler.start()
                    reps = max(10, int(seconds * 1e3 / best))
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(reps):
                        fn()
                    e1.record()
                    e1.synchronize()
                    clocks = sampler.stop()
                    out[key] = {"burst": round(ops / (best * 1e-3) / 1e12, 1),
                                "sustained": round(ops * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1),
                                "unit": "TOP/s" if key == "int8" else "TFLOP/s", "shape": "8192^3",
                                "sm_mhz_sustained": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}
                except Exception as e:  # the yardstick is missing: say so, keep the run
                    out[key] = {"error": str(e)[:200]}
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        del a8, b8, a32, b32
        torch.cuda.empty_cache()
    return out


def tensor_peak(peaks, lib_peaks, kind):
    """(peak, source) for a tensor-bound fraction: the measured library GEMM of that type where
    it could be measured, else the multiple of the measured bf16 GEMM that the tensor core's
    relative rates imply (int8 2 x, tf32 1/2 x)."""
    m = (lib_peaks or {}).get(kind, {})
    if "burst" in m:
        return m["burst"], "measured %s library GEMM 8192^3, burst (sustained %.0f)" % (kind, m["sustained"])
    factor = 2.0 if kind == "int8" else 0.5
    return factor * peaks["bf16_tflops"], "%g x %s bf16 burst (no %s yardstick)" % (factor, peaks["source"], kind)


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


class RawContext:
    """Event timing and launch counters on an mb_context owned by someone else."""

    def __init__(self, handle):
        import mace_b200
        self.L = mace_b200.lib()
        self.h = ctypes.c_void_p(handle)

    def event(self):
        e = ctypes.c_void_p()
        assert self.L.mb_event_create(self.h, ctypes.byref(e)) == 0
        return e

    def record(self, e):
        assert self.L.mb_event_record(self.h, e) == 0

    def elapsed_ms(self, a, b):
        ms = ctypes.c_float()
        assert self.L.mb_event_elapsed_ms(self.h, a, b, ctypes.byref(ms)) == 0
        return float(ms.value)

    def sync(self):
        rc = self.L.mb_stream_sync(self.h)
        if rc != 0:
            raise RuntimeError(self.L.mb_last_error(self.h).decode())

    @property
    def launches(self):
        return int(self.L.mb_launch_count(self.h))

    @property
    def launches_tensor_core(self):
        return int(self.L.mb_launch_count_tensor_core(self.h))

    def pinned(self, nbytes):
        p = ctypes.c_void_p()
        assert self.L.mb_host_alloc(self.h, int(nbytes), ctypes.byref(p)) == 0
        return np.ctypeslib.as_array((ctypes.c_uint8 * int(nbytes)).from_address(p.value))


def init_dist(world, local):
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return dist


def max_over_ranks(dist, values):
    if dist is None:
        return values
    import torch
    t = torch.tensor(values, device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


# --------------------------------------------------------------------------------------
# workload: uint8 GEMM 4096^3
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
        self.bytes_per_step = M * K + K * N + M * N  # algorithmic bytes of one launch (uint8)

    def quant(self, orc):
        # output scale for a +-4 sigma accumulator range (sum of K products of centred bytes)
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


def time_gemm(ctx, orc, wl, steps, warmup, rank=0):
    """Device-resident timing of the GEMM workload; returns (ms_per_step, sets, quant, n_sets)."""
    mult, shift, zp_c = wl.quant(orc)
    n_sets = max(2, int(np.ceil(1.5 * L2_BYTES / wl.bytes_per_step)))
    sets = []
    for i in range(n_sets):
        A, B = wl.host_inputs(1000 * rank + i)
        sets.append((ctx.upload(A), ctx.upload(B), ctx.alloc(wl.M * wl.N)))

    def step(i):
        dA, dB, dC = sets[i % n_sets]
        ctx.gemm_u8(dA, dB, None, dC, 1, wl.M, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)

    for i in range(max(warmup, 3)):
        step(i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for i in range(steps):
        step(i)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1)
    return ms / steps, sets, (mult, shift, zp_c), n_sets, step


def run_gemm(args, rank, world):
    import mace_b200
    from oracle import pyoracle as orc  # quantization parameters and the cpu_baseline leg only
    local = int(os.environ.get("LOCAL_RANK", rank))
    ctx = mace_b200.Context(local)
    size = int(getattr(args, "gemm_size", 4096) or 4096)
    wl = GemmWorkload(size, size, size)
    if size != 4096:
        wl.name = "gemm_u8_%d" % size
    dist = init_dist(world, local)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    _, sets, (mult, shift, zp_c), n_sets, step = time_gemm(ctx, orc, wl, 3, args.warmup, rank)
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

    hA, hB, hC = ctx.host_alloc(wl.M * wl.K), ctx.host_alloc(wl.K * wl.N), ctx.host_alloc(wl.M * wl.N)
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
    ms, e2e_ms = max_over_ranks(dist, [ms, e2e_ms])

    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        value = world * wl.ops_per_step / (ms_per_step * 1e-3) / 1e12
        e2e_val = world * wl.ops_per_step / (e2e_ms / e2e_steps * 1e-3) / 1e12
        peak, peak_src = tensor_peak(peaks, lib_peaks(local), "int8")
        achieved = wl.ops_per_step / (ms_per_step * 1e-3) / 1e12
        result = {
            "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(n_sets), parallelism="replicas only (dp%d)" % world),
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2),
                         "peak": round(peak, 1), "unit": "TOP/s",
                         "frac": round(achieved / peak, 4),
                         "traffic": NCU_TRAFFIC["gemm_u8_4096"] if size == 4096 else None,
                         "peak_source": peak_src,
                         "frac_of_2x_bf16_burst": round(achieved / (2.0 * peaks["bf16_tflops"]), 4),
                         "kernel": "gemm_u8_tc_kernel<256> (step also holds the operand-sum kernel)"},
            "e2e": {"value": round(e2e_val, 3), "unit": wl.unit,
                    "h2d_bytes_per_step": wl.M * wl.K + wl.K * wl.N,
                    "d2h_bytes_per_step": wl.M * wl.N},
            "gpu_launches": launches, "gpu_launches_tensor_core": launches_tc,
            "clocks": clocks,
        }
        result["cpu_baseline"] = gemm_cpu_baseline(wl, orc, mult, shift, zp_c, steps=2)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return result


def gemm_cpu_baseline(wl, orc, mult, shift, zp_c, steps):
    """The oracle (a port of the reference's CPU arithmetic) on this box's host cores."""
    A, B = wl.host_inputs(0)
    rows = min(wl.M, 1024)  # bounded sample: the first 1024 rows of A against the whole B
    threads = orc.set_threads(0)
    orc.gemm_u8(A[:64], B, None, 1, 64, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.gemm_u8(A[:rows], B, None, 1, rows, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
    dt = (time.perf_counter() - t0) / steps
    return {"value": round(2.0 * rows * wl.N * wl.K / dt / 1e12, 5), "unit": wl.unit,
            "cores": threads, "kind": "port",
            "sample": "%d of %d rows of A against all of B, %d passes" % (rows, wl.M, steps)}


# --------------------------------------------------------------------------------------
# workload: quantized MobileNet-v1, batch 64 per GPU
# --------------------------------------------------------------------------------------

BATCH = 64


def mobilenet_layer_bytes(layers, batch):
    """Algorithmic bytes per layer: input + output activation (uint8) + weights + int32 bias."""
    out = {}
    h, c = 224, 3
    for L in layers:
        if L["kind"] == "conv":
            o, kh, kw, _ = L["w"].shape
            ho = (h - 1) // L["stride"] + 1
            out[L["name"]] = batch * (h * h * c + ho * ho * o) + L["w"].size + 4 * o
            h, c = ho, o
        elif L["kind"] == "dw":
            ho = (h - 1) // L["stride"] + 1
            out[L["name"]] = batch * (h * h * c + ho * ho * c) + 9 * c + 4 * c
            h = ho
        elif L["kind"] == "pool":
            out[L["name"]] = batch * (h * h * c + c)
            h = 1
        else:
            out[L["name"]] = L["w"].size + batch * (1024 + 1000) + 4000
    return out


LIB_PEAKS = None  # library_tensor_peaks() of this process, once measured


def lib_peaks(local):
    global LIB_PEAKS
    if LIB_PEAKS is None:
        LIB_PEAKS = library_tensor_peaks(local)
    return LIB_PEAKS


class MobilenetRig:
    """One engine of the quantized MobileNet at a given per-GPU batch, with rotating pinned host
    inputs, and the two timed loops of the benchmark."""

    def __init__(self, mn, hostapi, layers, batch, local, rank, n_inputs=16, opts=()):
        self.mn, self.batch, self.n_inputs = mn, batch, n_inputs
        self.eng = mn.build_engine(hostapi, layers, batch, device=local)
        self.ctx = RawContext(self.eng.context)
        for item in opts:  # library switches for A/B runs (mb_set_option), e.g. --opt dw_tma=0
            name, _, value = item.partition("=")
            assert self.ctx.L.mb_set_option(self.ctx.h, name.encode(), int(value)) == 0, "unknown option " + item
        # rotate the engine over several input tensors so that consecutive steps do not find
        # their input in L2; activations (51 MB at the widest layer of batch 64) stream through
        # L2 on their own
        self.inputs = [mn.random_images(batch, seed=100 * rank + i) for i in range(n_inputs)]
        self.hin = self.ctx.pinned(self.inputs[0].nbytes * n_inputs).reshape(n_inputs, -1)
        for i, x in enumerate(self.inputs):
            self.hin[i] = x.ravel()
        self.houts = [self.ctx.pinned(batch * mn.NUM_CLASSES) for _ in range(2)]

    def warm_and_capture(self, warmup, graph=True, plan=False):
        mem = None
        for i in range(max(warmup, 3)):
            self.eng.write("input", self.inputs[i % self.n_inputs])
            self.eng.run(sync=False)
            if i == 0 and plan:
                self.eng.sync()
                mem = self.eng.plan_memory()
        if graph:
            self.eng.sync()
            self.eng.capture()  # the chain is replayed from one CUDA graph from here on
            self.eng.run(sync=False)
        return mem

    def timed_resident(self, steps):
        """Device-timed replays on the input the last (untimed) copy left in HBM: the input is
        1.5 % of the bytes a step moves, the rest (activations) exceeds L2 at batch 64."""
        ctx = self.ctx
        e0, e1 = ctx.event(), ctx.event()
        ctx.record(e0)
        for _ in range(steps):
            self.eng.run(sync=False)
        ctx.record(e1)
        return ctx.elapsed_ms(e0, e1)

    def e2e_loop(self, n, first, gather):
        """Pinned host input -> H2D -> chain -> D2H logits, every step, pipelined two deep: the
        upload of step i + 1 (upload stream, two staging buffers) overlaps the chain of step i,
        and the host takes delivery of step i - 1's logits (waits for their copy) after it has
        enqueued step i.  With several ranks the gather of the logits is enqueued behind every
        step (AsyncRowGather: a side stream, no host wait).  The region ends when the last logits
        -- and the last gather -- are in host memory."""
        prev = None
        for i in range(first, first + n):
            slot = self.eng.run_host_pipelined("input", self.hin[i % self.n_inputs], "fc", self.houts[i & 1])
            if gather is not None:
                gather.enqueue()
            if prev is not None:
                self.eng.wait_slot(prev)
            prev = slot
        self.eng.wait_slot(prev)
        if gather is not None:
            gather.wait()
        self.eng.sync()

    def make_gather(self, dist, world):
        if dist is None:
            return None
        from mace_b200.sharding import AsyncRowGather, torch_view
        import mace_b200
        ptr, nbytes = self.eng.device_ptr("fc")
        assert nbytes == self.batch * self.mn.NUM_CLASSES
        rows = torch_view(ptr, (self.batch, self.mn.NUM_CLASSES))
        stream = mace_b200.lib().mb_stream(ctypes.c_void_p(self.eng.context))
        return AsyncRowGather(dist, self.batch * world, rows, stream)

    def close(self):
        self.eng.close()


def h2d_rate(ctx, src_row, dist):
    """GB/s of this rank's uploads from pinned host memory with every rank copying at once
    (the slowest rank's figure): what the host's PCIe / memory path gives each GPU."""
    L = ctx.L
    nbytes = int(src_row.nbytes)
    dst = ctypes.c_void_p()
    assert L.mb_malloc(ctx.h, nbytes, ctypes.byref(dst)) == 0
    src = ctypes.c_void_p(src_row.ctypes.data)
    for _ in range(3):
        L.mb_memcpy_h2d(ctx.h, dst, src, nbytes)
    ctx.sync()
    if dist is not None:
        dist.barrier()
    reps = 20
    t0 = time.perf_counter()
    for _ in range(reps):
        L.mb_memcpy_h2d(ctx.h, dst, src, nbytes)
    ctx.sync()
    dt = time.perf_counter() - t0
    dt = max_over_ranks(dist, [dt])[0]
    L.mb_free(ctx.h, dst)
    return reps * nbytes / dt / 1e9


def run_mobilenet(args, rank, world):
    import mace_b200
    from mace_b200 import hostapi
    from oracle import pyoracle as orc  # model construction (quantization math) and cpu_baseline
    from mace_b200.harness import mobilenet_v1 as mn
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist = init_dist(world, local)
    layers = mn.build(orc, seed=0)
    rig = MobilenetRig(mn, hostapi, layers, BATCH, local, rank, opts=args.opt)
    eng, ctx = rig.eng, rig.ctx

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    mem = rig.warm_and_capture(args.warmup, graph=not args.no_graph, plan=args.plan)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.01)
    l0, ltc0 = ctx.launches, ctx.launches_tensor_core
    ms = rig.timed_resident(args.steps)
    barrier()
    launches, launches_tc = ctx.launches - l0, ctx.launches_tensor_core - ltc0
    clocks = sampler.stop() if rank == 0 else None
    if args.profile:
        rig.close()
        return None

    # per-operator device times inside a graph replay (event nodes between the operators of a
    # second recorded graph): they add up to the replayed step
    per_op = dict(eng.run_profiled_graph(replays=5))

    gather = rig.make_gather(dist, world)
    rig.e2e_loop(4, 0, gather)
    barrier()
    e2e_steps = max(4, min(args.steps, 50))
    t0 = time.perf_counter()
    rig.e2e_loop(e2e_steps, 4, gather)
    e2e_ms = (time.perf_counter() - t0) * 1e3  # host clock around enqueue ... last logits on the host
    barrier()
    gathered_ok = None
    if gather is not None and rank == 0:  # the gathered rows of the last step: rank 0's own rows must be in place
        full = gather.wait().numpy()
        gathered_ok = bool(np.array_equal(full[:BATCH].ravel(), rig.houts[(4 + e2e_steps - 1) & 1]))
    h2d_gbs = h2d_rate(ctx, rig.hin[0], dist)
    ms, e2e_ms = max_over_ranks(dist, [ms, e2e_ms])

    # strong scaling: the configuration's own batch of 64 split over the ranks
    strong = None
    if world > 1 and BATCH % world == 0:
        srig = MobilenetRig(mn, hostapi, layers, BATCH // world, local, rank, opts=args.opt)
        srig.warm_and_capture(args.warmup, graph=not args.no_graph)
        barrier()
        s_ms = srig.timed_resident(args.steps)
        barrier()
        sg = srig.make_gather(dist, world)
        srig.e2e_loop(4, 0, sg)
        barrier()
        t0 = time.perf_counter()
        srig.e2e_loop(e2e_steps, 4, sg)
        s_e2e = (time.perf_counter() - t0) * 1e3
        barrier()
        s_ms, s_e2e = max_over_ranks(dist, [s_ms, s_e2e])
        strong = {"global_batch": BATCH, "batch_per_gpu": BATCH // world,
                  "value": round(BATCH / (s_ms / args.steps * 1e-3), 1), "unit": "images/s",
                  "ms_per_step": round(s_ms / args.steps, 4),
                  "e2e": {"value": round(BATCH / (s_e2e / e2e_steps * 1e-3), 1), "unit": "images/s"}}
        srig.close()

    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        value = world * BATCH / (ms_per_step * 1e-3)
        e2e_val = world * BATCH / (e2e_ms / e2e_steps * 1e-3)
        lbytes = mobilenet_layer_bytes(layers, BATCH)
        # group operator times by kernel family
        fam = {"dw": ["dwconv3x3_u8_tma_kernel", 0.0, 0], "pw": ["gemm_u8_tc_kernel (pointwise; the depth-32 first one on conv_u8_stem_mma_kernel)", 0.0, 0],
               "stem": ["conv_u8_stem_mma_kernel", 0.0, 0], "pool": ["avgpool_u8_c4_kernel", 0.0, 0],
               "fc": ["gemm_u8_tc_kernel (FullyConnected, float rule)", 0.0, 0]}
        for label, t in per_op.items():
            name = label.split(":")[1]
            key = "dw" if name.startswith("dw") else "pw" if name.startswith("pw") else name
            fam[key][1] += t
            fam[key][2] += lbytes[name]
        # The event nodes between the operators serialise the graph (no overlap of one kernel's tail
        # with the next one's prologue) and add their own latency, so the per-operator times add up
        # to more than the replayed step: each family's SHARE of that sum is applied to the timed
        # step, which makes the families add up to ms_per_step.
        total_prof = sum(v[1] for v in fam.values())
        scale = ms_per_step / total_prof
        dom = max(fam.values(), key=lambda v: v[1])
        achieved = dom[2] / (dom[1] * scale * 1e-3) / 1e9
        achieved_serialised = dom[2] / (dom[1] * 1e-3) / 1e9
        total_bytes = sum(lbytes.values())
        result = {
            "metric": "quantized_mobilenet_v1_images_per_s", "value": round(value, 1),
            "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
            "data": "synthetic",
            "config": {"workload": "mobilenet_v1_u8_b64", "batch_per_gpu": BATCH,
                       "global_batch": BATCH * world, "image": "224x224x3 uint8 NHWC",
                       "weights": "He-normal, per-tensor uint8 (non_zero), seed 0",
                       "parallelism": "dp%d: batch sharded, weights replicated, final logits gather only" % world,
                       "launch": "per-operator launches" if args.no_graph else "CUDA graph replay",
                       "l2": ("activations of one step (%.0f MB) exceed L2" % (total_bytes / 1e6)) if mem is None else
                       ("activations of one step (%.0f MB) pass through shared buffers of %.0f MB in total"
                        % (total_bytes / 1e6, mem[1] / 1e6))},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4),
                         "traffic": NCU_TRAFFIC["mobilenet_dw" if dom is fam["dw"] else "mobilenet_pw"]
                         if dom in (fam["dw"], fam["pw"]) else None,
                         "peak_source": "%s copy bandwidth" % peaks["source"],
                         "kernel": dom[0],
                         "kernel_share_of_step": round(dom[1] / total_prof, 3),
                         "kernel_ms_in_step": round(dom[1] * scale, 4),
                         "achieved_serialised": round(achieved_serialised, 1),
                         "frac_serialised": round(achieved_serialised / peaks["hbm_gbs"], 4),
                         "algorithmic_bytes_per_step": dom[2]},
            "model_hbm": {"algorithmic_bytes_per_step": total_bytes,
                          "achieved_gbs": round(total_bytes / (ms_per_step * 1e-3) / 1e9, 1),
                          "frac_of_peak": round(total_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)},
            "kernel_families_ms": dict({v[0]: round(v[1] * scale, 4) for v in fam.values()},
                                       how="shares from event nodes between the operators of a replayed graph "
                                           "(serialised sum %.4f ms), applied to the timed step" % total_prof),
            "kernel_families_ms_serialised": {v[0]: round(v[1], 4) for v in fam.values()},
            "e2e": {"value": round(e2e_val, 1), "unit": "images/s",
                    "h2d_bytes_per_step": int(rig.inputs[0].nbytes),
                    "d2h_bytes_per_step": BATCH * mn.NUM_CLASSES},
            "h2d_gbs_per_rank": round(h2d_gbs, 2),
            "gpu_launches": launches, "gpu_launches_tensor_core": launches_tc, "clocks": clocks,
        }
        if dist is not None:
            result["gather"] = {"kind": "all_gather_into_tensor on a side stream, one per step, rank 0 copies "
                                        "the rows to pinned host memory", "rows_in_place": gathered_ok}
        if strong is not None:
            result["strong_scaling"] = strong
        elif world == 1:
            result["strong_scaling"] = {"global_batch": BATCH, "batch_per_gpu": BATCH, "value": round(value, 1),
                                        "unit": "images/s", "ms_per_step": round(ms_per_step, 4),
                                        "e2e": {"value": round(e2e_val, 1), "unit": "images/s"}}
    rig.close()
    if rank == 0:
        lp = lib_peaks(local)
        result["tensor_peaks_measured"] = lp
        # the other half of the metric: u8 GEMM TOPS on the 4096^3 MatMul
        gctx = mace_b200.Context(local)
        gwl = GemmWorkload()
        gms, _, _, _, _ = time_gemm(gctx, orc, gwl, 30, 5)
        gtops = gwl.ops_per_step / (gms * 1e-3) / 1e12
        ipeak, isrc = tensor_peak(peaks, lp, "int8")
        result["u8_gemm"] = {"workload": gwl.name, "value": round(gtops, 2), "unit": "TOPS",
                             "ms_per_step": round(gms, 5),
                             "frac_of_int8_peak": round(gtops / ipeak, 4), "int8_peak": ipeak, "peak_source": isrc,
                             "frac_of_2x_bf16_peak": round(gtops / (2 * peaks["bf16_tflops"]), 4)}
        gctx.close()
        # the same network as a converted-model file through the model-level API (NetDef bytes +
        # weights blob -> CreateMaceEngineFromProto; one synchronous MaceEngine::Run per step on
        # pinned host buffers: upload, graph replay, download, wait)
        if world == 1:
            from mace_b200.harness import netdef_wire
            writer = netdef_wire.NetDefWriter(quantized=True, name="mobilenet_v1_u8")
            mn.build_engine(netdef_wire.WriterModule(hostapi, writer), layers, BATCH)
            writer.add_output("fc", (BATCH, 1, 1, mn.NUM_CLASSES), data_type=netdef_wire.DT_UINT8)
            model = hostapi.Model(writer.netdef(), writer.weights(), device=local, plan_memory=True, cuda_graph=True)
            mctx = RawContext(model.context)
            mout = mctx.pinned(BATCH * mn.NUM_CLASSES).reshape(BATCH, 1, 1, mn.NUM_CLASSES)
            minp = mctx.pinned(rig.inputs[0].nbytes * 4).reshape((4,) + rig.inputs[0].shape)
            for i in range(4):
                minp[i] = rig.inputs[i]

            def model_step(i):
                return model.run({"input": (minp[i % 4], hostapi.DF_NHWC)}, {"fc": (mout, hostapi.DF_NHWC)})

            for i in range(4):
                model_step(i)
            msteps = max(4, min(args.steps, 50))
            t0 = time.perf_counter()
            for i in range(msteps):
                model_step(4 + i)
            mms = (time.perf_counter() - t0) * 1e3 / msteps
            result["e2e_model_api"] = {"value": round(BATCH / (mms * 1e-3), 1), "unit": "images/s",
                                       "ms_per_step": round(mms, 4), "graph": model.captured,
                                       "call": "MaceEngine::Run on a model file, synchronous, pinned host buffers"}
            model.close()
        # CPU baseline: the oracle chain on this box's host cores, full batches
        threads = orc.set_threads(0)
        x = rig.inputs[0]
        mn.oracle_forward(orc, layers, x[:4])
        t0 = time.perf_counter()
        passes = 2
        for _ in range(passes):
            mn.oracle_forward(orc, layers, x)
        dt = (time.perf_counter() - t0) / passes
        result["cpu_baseline"] = {"value": round(BATCH / dt, 2), "unit": "images/s",
                                  "cores": threads, "kind": "port",
                                  "sample": "%d full batches of %d images" % (passes, BATCH)}
        if world == 1 and not args.no_extras:
            result["configs"] = other_config_records(args, rank)
    if dist is not None:
        dist.destroy_process_group()
    return result


def other_config_records(args, rank):
    """Compact records of the other benchmark configurations (the 1024^3 MatMul, the Winograd
    convolution, the K = N = 4096 sweep with the batched MatMul and the GEMV, ResNet-50 at batch
    256), each timed with its own CUDA events over >= 20 steps, for the default line."""
    import copy
    sub = copy.copy(args)
    sub.steps, sub.warmup, sub.profile = max(20, min(args.steps, 50)), max(args.warmup, 3), False
    out = {}

    def pick(res, keys):
        return {k: res[k] for k in keys if k in res}

    try:
        sub.gemm_size = 1024
        r = run_gemm(sub, rank, 1)
        out["gemm_u8_1024"] = dict(pick(r, ("value", "unit", "ms_per_step")), frac=r["roofline"]["frac"],
                                   peak=r["roofline"]["peak"], e2e=r["e2e"]["value"],
                                   cpu_baseline=r["cpu_baseline"]["value"])
    except Exception as e:
        out["gemm_u8_1024"] = {"error": str(e)[:200]}
    sub.gemm_size = 4096
    try:
        r = run_winograd(sub, rank, 1)
        out["winograd_f32_cfg1"] = dict(pick(r, ("value", "unit", "ms_per_step")), hbm_frac=r["roofline"]["frac"],
                                        e2e=r["e2e"]["value"], cpu_baseline=r["cpu_baseline"]["value"])
    except Exception as e:
        out["winograd_f32_cfg1"] = {"error": str(e)[:200]}
    try:
        r = run_sweep(sub, rank, 1)
        out["gemm_u8_sweep"] = r["cases"]
    except Exception as e:
        out["gemm_u8_sweep"] = {"error": str(e)[:200]}
    try:
        r = run_resnet(sub, rank, 1)
        out["resnet50_f32_b256"] = dict(pick(r, ("value", "unit", "ms_per_step")), tensor_frac=r["roofline"]["frac"],
                                        tflops=r["roofline"]["achieved"], e2e=r["e2e"]["value"],
                                        cpu_baseline=r["cpu_baseline"]["value"])
    except Exception as e:
        out["resnet50_f32_b256"] = {"error": str(e)[:200]}
    return out


# --------------------------------------------------------------------------------------
# workload: fp32 3x3 Conv2D by Winograd (input [32,64,56,56], filter [64,64,3,3], SAME)
# --------------------------------------------------------------------------------------

def run_winograd(args, rank, world):
    import mace_b200
    from oracle import pyoracle as orc  # cpu_baseline leg only
    local = int(os.environ.get("LOCAL_RANK", rank))
    ctx = mace_b200.Context(local)
    dist = init_dist(world, local)
    N, C, H, W, O = 32, 64, 56, 56, 64
    rng = np.random.Generator(np.random.PCG64(rank))
    f = (rng.standard_normal((O, C, 3, 3)) * np.sqrt(2.0 / (9 * C))).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.01).astype(np.float32)
    n_sets = 6  # 6 x (25.7 MB in + 25.7 MB out) = 308 MB > L2
    xs = [rng.random((N, C, H, W), dtype=np.float32) for _ in range(n_sets)]
    dxs = [ctx.upload(x) for x in xs]
    dos = [ctx.alloc(N * O * H * W * 4) for _ in range(n_sets)]
    df, db = ctx.upload(f), ctx.upload(bias)
    dU = ctx.alloc(64 * O * C * 4)
    ctx.winograd_transform_filter(df, dU, C, O, 6)  # cached per weight, as the delegator does

    def step(i):
        ctx.winograd_f32(dxs[i % n_sets], df, db, dos[i % n_sets], N, C, H, W, O, (1, 1), (H, W),
                         transformed=dU)

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
    hx, ho = ctx.host_alloc(xs[0].nbytes), ctx.host_alloc(N * O * H * W * 4)
    hx[:] = xs[0].view(np.uint8).ravel()

    def e2e_step():
        ctx.h2d(dxs[0], hx)
        step(0)
        ctx.d2h(ho, dos[0])

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
    ms, e2e_ms = max_over_ranks(dist, [ms, e2e_ms])
    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        direct_flops = 2.0 * N * O * C * 9 * H * W
        alg_bytes = 4 * (N * C * H * W + N * O * H * W + O * C * 9 + O)
        value = world * direct_flops / (ms_per_step * 1e-3) / 1e12
        achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
        result = {
            "metric": "fp32_conv3x3_winograd_direct_equivalent_tflops", "value": round(value, 2),
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "winograd_f32_cfg1", "input": [N, C, H, W], "filter": [O, C, 3, 3],
                       "padding": "SAME", "tile": "F(6x6,3x3)", "executed_gemm_flops": 2.0 * 64 * O * C * N * 100,
                       "l2": "rotating %d input/output sets (%.0f MB > L2)" % (n_sets, n_sets * 51.4),
                       "parallelism": "dp%d: batch sharded, filter replicated" % world},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                         "traffic": NCU_TRAFFIC["winograd_f32_cfg1"],
                         "peak_source": "%s copy bandwidth" % peaks["source"],
                         "kernel": "whole call: wino_input_kernel + gemm_f32_tc_kernel + wino_output_kernel",
                         "algorithmic_bytes_per_step": alg_bytes},
            "e2e": {"value": round(world * direct_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, 2),
                    "unit": "TFLOP/s", "h2d_bytes_per_step": int(xs[0].nbytes),
                    "d2h_bytes_per_step": N * O * H * W * 4},
            "gpu_launches": launches, "gpu_launches_tensor_core": launches_tc, "clocks": clocks,
        }
        threads = orc.set_threads(0)
        sample_n = 4
        orc.winograd_f32(xs[0][:1], f, bias, (1, 1), (H, W), 0, 0.0, 0.0)
        t0 = time.perf_counter()
        orc.winograd_f32(xs[0][:sample_n], f, bias, (1, 1), (H, W), 0, 0.0, 0.0)
        dt = time.perf_counter() - t0
        result["cpu_baseline"] = {"value": round(direct_flops * sample_n / N / dt / 1e12, 4),
                                  "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                  "sample": "%d of %d images, one pass" % (sample_n, N)}
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return result


# --------------------------------------------------------------------------------------
# workload: ResNet-50 v1, fp32 NCHW, batch 256 per GPU
# --------------------------------------------------------------------------------------

def resnet_kind(node):
    if node["op"] == "conv":
        if node["k"] == 7:
            return "stem 7x7 s2 (im2col + gemm_f32_tc_kernel)"
        if node["k"] == 3:
            return "3x3 s1 (Winograd: wino_input + gemm_f32_tc_kernel + wino_output)"
        if node["stride"] == 2:
            return "1x1 s2 (pixel gather + gemm_f32_tc_kernel)"
        return "1x1 s1 (gemm_f32_tc_kernel)"
    return {"maxpool": "max pool", "avgpool": "avg pool", "add": "eltwise sum", "relu": "activation",
            "fc": "fully connected"}[node["op"]]


def run_resnet(args, rank, world):
    import mace_b200  # noqa: F401  (fails loudly when the device library is missing)
    from mace_b200 import hostapi
    from oracle import pyoracle as orc  # cpu_baseline leg only
    from mace_b200.harness import resnet50 as rn
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist = init_dist(world, local)
    batch = args.batch or 256
    nodes, weights = rn.build(seed=0)
    eng = rn.build_engine(hostapi, nodes, weights, batch, device=local)
    # one gather for the two stride-2 1x1 convolutions that open a stage (shortcut and branch2a)
    shared = 0 if args.no_fuse else eng.share_subsampled_inputs()
    merged = 0 if args.no_fuse else eng.fuse_activations()  # residual sum + ReLU in one pass
    ctx = RawContext(eng.context)
    x = rn.random_images(batch, seed=100 + rank)
    hin = ctx.pinned(x.nbytes)
    hin[:] = x.view(np.uint8).ravel()
    hout = ctx.pinned(batch * rn.NUM_CLASSES * 4)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    eng.write("input", x)
    eng.run()
    merged_conv = 0 if args.no_fuse else eng.fuse_residual_sums()  # ... and into the 1x1 conv before it
    mem = None
    if not args.no_plan:  # activation memory shared between tensors with disjoint lifetimes
        mem = eng.plan_memory()
    for i in range(max(args.warmup, 3)):
        eng.run(sync=False)
    if not args.no_graph:
        eng.sync()
        eng.capture()
        eng.run(sync=False)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.01)
    l0, ltc0 = ctx.launches, ctx.launches_tensor_core
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for i in range(args.steps):
        eng.run(sync=False)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1)
    barrier()
    launches, launches_tc = ctx.launches - l0, ctx.launches_tensor_core - ltc0
    clocks = sampler.stop() if rank == 0 else None
    if args.profile:
        eng.close()
        return None
    kinds = {n["name"]: resnet_kind(n) for n in nodes}
    fam = {}
    prof_runs = 3
    for _ in range(prof_runs):
        for label, t in eng.run_profiled(max_ops=512):
            k = kinds.get(label.split(":", 1)[-1], label)
            if label.startswith("Subsample:"):
                k = "1x1 s2 (pixel gather + gemm_f32_tc_kernel)"
            fam[k] = fam.get(k, 0.0) + t / prof_runs

    # pipelined end-to-end calls (see run_mobilenet): the next batch's upload overlaps this
    # batch's run; two pinned host input and output buffers rotate
    hins = [hin, ctx.pinned(x.nbytes)]
    hins[1][:] = rn.random_images(batch, seed=200 + rank).view(np.uint8).ravel()
    houts = [hout, ctx.pinned(batch * rn.NUM_CLASSES * 4)]

    def gather(call):
        slot, buf = call
        eng.wait_slot(slot)
        from mace_b200.sharding import gather_rows
        gather_rows(dist, houts[buf].view(np.float32).reshape(batch, rn.NUM_CLASSES), batch * world,
                    device="cuda")

    def e2e_loop(n):
        prev = None
        for i in range(n):
            slot = eng.run_host_pipelined("input", hins[i & 1], "fc", houts[i & 1])
            if dist is not None and prev is not None:
                gather(prev)
            prev = (slot, i & 1)
        if dist is not None:
            gather(prev)
        eng.sync()

    e2e_loop(2)
    barrier()
    e2e_steps = max(4, min(args.steps, 10))
    t0 = time.perf_counter()
    e2e_loop(e2e_steps)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    ms, e2e_ms = max_over_ranks(dist, [ms, e2e_ms])
    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        macs = rn.macs_per_image(nodes)
        value = world * batch / (ms_per_step * 1e-3)
        tflops = 2.0 * macs * batch / (ms_per_step * 1e-3) / 1e12
        tf32_peak, tf32_src = tensor_peak(peaks, lib_peaks(local), "tf32")
        alg_bytes = rn.activation_bytes(nodes, batch)
        result = {
            "metric": "fp32_resnet50_images_per_s", "value": round(value, 1), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "resnet50_f32_b256", "batch_per_gpu": batch, "global_batch": batch * world,
                       "image": "224x224x3 fp32 NCHW", "weights": "He-normal, seed 0",
                       "macs_per_image": macs,
                       "parallelism": "dp%d: batch sharded, weights replicated, final logits gather only" % world,
                       "launch": "operator by operator" if args.no_graph else "CUDA graph replay",
                       "merged_sum_relu_pairs": merged, "sums_merged_into_convolutions": merged_conv,
                       "shared_stride2_gathers": shared,
                       "activation_memory_gb": None if mem is None else
                       {"one_buffer_per_tensor": round(mem[0] / 1e9, 2), "planned": round(mem[1] / 1e9, 2)},
                       "l2": "activations of one step (%.1f GB) exceed L2" % (alg_bytes / 1e9)},
            "roofline": {"bound": "tensor", "achieved": round(tflops, 2), "peak": round(tf32_peak, 1),
                         "unit": "TFLOP/s", "frac": round(tflops / tf32_peak, 4), "traffic": None,
                         "peak_source": tf32_src + "; the fp32 GEMMs run three tf32 MMAs per product (hi/lo "
                                        "split), so a third of it is the ceiling for direct-equivalent flops "
                                        "outside Winograd",
                         "kernel": "whole step (gemm_f32_tc_kernel dominates)",
                         "direct_equivalent_flops_per_step": 2.0 * macs * batch},
            "model_hbm": {"algorithmic_bytes_per_step": alg_bytes,
                          "achieved_gbs": round(alg_bytes / (ms_per_step * 1e-3) / 1e9, 1),
                          "frac_of_peak": round(alg_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)},
            "operator_kinds_ms": {k: round(v, 4) for k, v in sorted(fam.items(), key=lambda kv: -kv[1])},
            "e2e": {"value": round(world * batch / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "images/s",
                    "h2d_bytes_per_step": int(x.nbytes), "d2h_bytes_per_step": batch * rn.NUM_CLASSES * 4},
            "gpu_launches": launches, "gpu_launches_tensor_core": launches_tc, "clocks": clocks,
        }
        threads = orc.set_threads(0)
        sample_n = 2
        t0 = time.perf_counter()
        rn.oracle_forward(orc, nodes, weights, x[:sample_n])
        dt = time.perf_counter() - t0
        result["cpu_baseline"] = {"value": round(sample_n / dt, 3), "unit": "images/s", "cores": threads,
                                  "kind": "port", "sample": "%d images, one pass (direct fp32 convolutions)" % sample_n}
    eng.close()
    if dist is not None:
        dist.destroy_process_group()
    return result


# --------------------------------------------------------------------------------------
# workload: uint8 GEMM / GEMV sweep, K = N = 4096, M in {1, 16, 128, 4096}, batched 64 x 512^3
# --------------------------------------------------------------------------------------

def run_sweep(args, rank, world):
    import mace_b200
    from oracle import pyoracle as orc
    local = int(os.environ.get("LOCAL_RANK", rank))
    ctx = mace_b200.Context(local)
    dist = init_dist(world, local)
    peaks = measured_peaks()
    int8_peak, int8_src = tensor_peak(peaks, lib_peaks(local) if rank == 0 else None, "int8")
    rows = []

    def timed(fn, n):
        for i in range(max(args.warmup, 3)):
            fn(i)
        ctx.sync()
        e0, e1 = ctx.event(), ctx.event()
        ctx.record(e0)
        for i in range(n):
            fn(i)
        ctx.record(e1)
        return ctx.elapsed_ms(e0, e1) / n

    K = Nn = 4096
    n_sets = 10  # 10 x 16.8 MB of B > L2
    rng = np.random.Generator(np.random.PCG64(rank))
    Bs = [ctx.upload(rng.integers(0, 256, size=(K, Nn), dtype=np.uint8)) for _ in range(n_sets)]
    for M in (1, 16, 128, 4096):
        wl = GemmWorkload(M, Nn, K)
        mult, shift, zp_c = wl.quant(orc)
        dA = ctx.upload(rng.integers(0, 256, size=(M, K), dtype=np.uint8))
        dC = ctx.alloc(M * Nn)
        ms = timed(lambda i: ctx.gemm_u8(dA, Bs[i % n_sets], None, dC, 1, M, Nn, K, wl.zp_a, wl.zp_b,
                                         mult, shift, zp_c), args.steps)
        byts = M * K + K * Nn + M * Nn
        rows.append({"case": "M=%d" % M, "ms": round(ms, 5), "tops": round(2.0 * M * Nn * K / ms / 1e9, 2),
                     "gbs": round(byts / ms / 1e6, 1),
                     "frac_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4),
                     "frac_int8_peak": round(2.0 * M * Nn * K / ms / 1e9 / int8_peak, 4),
                     "frac_2x_bf16": round(2.0 * M * Nn * K / ms / 1e9 / (2 * peaks["bf16_tflops"]), 4)})
    # batched MatMul 64 x 512^3
    bA = [ctx.upload(rng.integers(0, 256, size=(64, 512, 512), dtype=np.uint8)) for _ in range(5)]
    bB = [ctx.upload(rng.integers(0, 256, size=(64, 512, 512), dtype=np.uint8)) for _ in range(5)]
    bC = ctx.alloc(64 * 512 * 512)
    wl = GemmWorkload(512, 512, 512)
    mult, shift, zp_c = wl.quant(orc)
    ms = timed(lambda i: ctx.gemm_u8(bA[i % 5], bB[i % 5], None, bC, 64, 512, 512, 512, wl.zp_a, wl.zp_b,
                                     mult, shift, zp_c), args.steps)
    rows.append({"case": "batch64_512^3", "ms": round(ms, 5), "tops": round(2.0 * 64 * 512 ** 3 / ms / 1e9, 2),
                 "gbs": round(3 * 64 * 512 * 512 / ms / 1e6, 1),
                 "frac_int8_peak": round(2.0 * 64 * 512 ** 3 / ms / 1e9 / int8_peak, 4),
                 "frac_2x_bf16": round(2.0 * 64 * 512 ** 3 / ms / 1e9 / (2 * peaks["bf16_tflops"]), 4)})
    # GEMV with the FullyConnected rule: weights [4096 x 4096], one vector
    Ws = [ctx.upload(rng.integers(0, 256, size=(1, 4096, 4096), dtype=np.uint8)) for _ in range(n_sets)]
    dx, dout = ctx.upload(rng.integers(0, 256, size=(1, 4096), dtype=np.uint8)), ctx.alloc(4096)
    ms = timed(lambda i: ctx.gemv_u8(Ws[i % n_sets], dx, None, dout, 1, 4096, 4096, 120, 128,
                                     np.float32(1e-5), 30, True), args.steps)
    gemv_gbs = 4096 * 4096 / ms / 1e6
    rows.append({"case": "gemv_4096x4096", "ms": round(ms, 5), "gbs": round(gemv_gbs, 1),
                 "frac_hbm": round(gemv_gbs / peaks["hbm_gbs"], 4)})
    # the same GEMV as it runs inside a network: ten calls on rotating matrices recorded into
    # one CUDA graph, so that the launch latency of a lone kernel is not part of the figure
    # ("weights": the matrices declared constant, as the Gemv delegator does for a tensor that
    # is_weight(): the kernel may then fetch its first bytes while the previous one still runs)
    L = mace_b200.lib()
    for const, label in ((0, "gemv_4096x4096_in_graph_of_%d"), (1, "gemv_4096x4096_weights_in_graph_of_%d")):
        ctx.set_option("gemv_lhs_const", const)
        ctx._check(L.mb_graph_begin(ctx.h))
        for i in range(n_sets):
            ctx.gemv_u8(Ws[i], dx, None, dout, 1, 4096, 4096, 120, 128, np.float32(1e-5), 30, True)
        graph = ctypes.c_void_p()
        ctx._check(L.mb_graph_end(ctx.h, ctypes.byref(graph)))
        ms = timed(lambda i: ctx._check(L.mb_graph_launch(ctx.h, graph)), max(3, args.steps // 2)) / n_sets
        ctx._check(L.mb_graph_destroy(ctx.h, graph))
        rows.append({"case": label % n_sets, "ms": round(ms, 5),
                     "gbs": round(4096 * 4096 / ms / 1e6, 1),
                     "frac_hbm": round(4096 * 4096 / ms / 1e6 / peaks["hbm_gbs"], 4)})
    ctx.set_option("gemv_lhs_const", 0)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    if rank != 0:
        return None
    big = [r for r in rows if r["case"] == "M=4096"][0]
    return {"metric": "u8_gemm_tops", "value": big["tops"], "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": big["ms"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
            "data": "synthetic",
            "config": {"workload": "gemm_u8_sweep", "K": K, "N": Nn,
                       "l2": "rotating %d B matrices (%.0f MB > L2)" % (n_sets, n_sets * 16.8),
                       "int8_peak": int8_peak, "int8_peak_source": int8_src,
                       "parallelism": "replicas only (dp%d)" % world},
            "cases": rows}


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path, timed on the host cores: the oracle
    port (the reference's own sources need NEON, gemmlowp, a TF-Lite fork and generated
    protobuf code, none of which exist here)."""
    if rank != 0:
        return None
    from oracle import pyoracle as orc
    threads = orc.set_threads(0)
    if args.workload == "gemm_u8_4096":
        wl = GemmWorkload()
        mult, shift, zp_c = wl.quant(orc)
        A, B = wl.host_inputs(0)
        rows = min(wl.M, 1024)
        orc.gemm_u8(A[:64], B, None, 1, 64, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
        steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(steps):
            orc.gemm_u8(A[:rows], B, None, 1, rows, wl.N, wl.K, wl.zp_a, wl.zp_b, mult, shift, zp_c)
        dt = (time.perf_counter() - t0) / steps
        value = round(2.0 * rows * wl.N * wl.K / dt / 1e12, 5)
        sample = "%d of %d rows of A against all of B per step" % (rows, wl.M)
        metric, unit, config = wl.metric, wl.unit, dict(wl.config(1), parallelism="host cores")
        ms_per_step = dt * 1e3 * wl.M / rows
    else:
        from mace_b200.harness import mobilenet_v1 as mn
        layers = mn.build(orc, seed=0)
        sample_n = BATCH  # the whole batch of the configuration, every step
        x = mn.random_images(sample_n, seed=0)
        mn.oracle_forward(orc, layers, x[:2])
        steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(steps):
            mn.oracle_forward(orc, layers, x)
        dt = (time.perf_counter() - t0) / steps
        value = round(sample_n / dt, 2)
        sample = "the full batch of %d images per step" % BATCH
        metric, unit = "quantized_mobilenet_v1_images_per_s", "images/s"
        config = {"workload": "mobilenet_v1_u8_b64", "batch_per_gpu": BATCH, "global_batch": BATCH,
                  "image": "224x224x3 uint8 NHWC",
                  "weights": "He-normal, per-tensor uint8 (non_zero), seed 0",
                  "parallelism": "host cores (%d threads), one process" % threads, "sample": sample}
        ms_per_step = dt * 1e3 * BATCH / sample_n
    return {"impl": "reference", "metric": metric, "value": value, "unit": unit,
            "n_gpus": world, "steps": steps, "warmup": 1, "ms_per_step": round(ms_per_step, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
            "data": "synthetic", "config": config,
            "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mobilenet_v1_u8_b64",
                    choices=["mobilenet_v1_u8_b64", "gemm_u8_4096", "winograd_f32_cfg1", "gemm_u8_sweep",
                             "resnet50_f32_b256"])
    ap.add_argument("--batch", type=int, default=0, help="images per GPU for resnet50_f32_b256 (default 256)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every operator separately instead of replaying a CUDA graph")
    ap.add_argument("--no-fuse", action="store_true",
                    help="resnet50_f32_b256: keep residual sums and their ReLUs as separate operators")
    ap.add_argument("--plan", action="store_true",
                    help="mobilenet_v1_u8_b64: share activation memory between layers (two buffers)")
    ap.add_argument("--no-plan", action="store_true",
                    help="resnet50_f32_b256: every activation tensor keeps its own buffer")
    ap.add_argument("--no-extras", action="store_true",
                    help="mobilenet_v1_u8_b64: skip the records of the other configurations")
    ap.add_argument("--gemm-size", type=int, default=4096, help="gemm_u8_4096: M = N = K (1024: config 0)")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=INT",
                    help="mobilenet_v1_u8_b64: a library option (mb_set_option) to set before the run; repeatable")
    ap.add_argument("--profile", action="store_true",
                    help="run only the device-resident timed loop (for ncu captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    # stdout carries the one JSON line and nothing else: whatever libraries print there (NCCL's
    # version banner, for one) is sent to stderr for the duration of the run
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        res = run_reference(args, rank, world)
    elif args.workload == "gemm_u8_4096":
        res = run_gemm(args, rank, world)
    elif args.workload == "winograd_f32_cfg1":
        res = run_winograd(args, rank, world)
    elif args.workload == "gemm_u8_sweep":
        res = run_sweep(args, rank, world)
    elif args.workload == "resnet50_f32_b256":
        res = run_resnet(args, rank, world)
    else:
        res = run_mobilenet(args, rank, world)
    sys.stdout.flush()
    if rank == 0 and res is not None:
        os.write(json_fd, (json.dumps(res) + "\n").encode())
    os.close(json_fd)


if __name__ == "__main__":
    main()
