"""Post-training quantization ranges from a run's log.

With the environment switch MACE_LOG_TENSOR_RANGE on, the sequential net logs one line
``Tensor range @@<tensor>@@<min>,<max>`` per operator output and run (the float model is run
over a set of calibration inputs).  This module turns such a log into one (min, max) per
tensor and into the uint8 scale / zero point the converter would store -- the arithmetic of
the reference's tools/python/quantize/quantize_stat.py:27-95 (percentile over the per-run
extremes, optional "enhance" mode that drops outlier runs while the range shrinks faster than
the share of runs it gives up) and tools/python/quantize/quantize_util.py:102-122
(adjust_range), written for this harness.
"""
import math

import numpy as np

MARK = "Tensor range @@"


def parse_ranges(lines):
    """-> ({tensor: ([mins], [maxs])}, [tensors in order of first appearance])."""
    ranges, order = {}, []
    for line in lines:
        at = line.find(MARK)
        if at < 0:
            continue
        fields = line[at + len(MARK):].split("@@")
        if len(fields) < 2:
            continue
        name = fields[0]
        lo, hi = (float(v) for v in fields[1].strip().split(","))
        if name not in ranges:
            ranges[name] = ([], [])
            order.append(name)
        ranges[name][0].append(lo)
        ranges[name][1].append(hi)
    return ranges, order


def overall_ranges(lines, percentile=0, enhance=False, enhance_ratio=10):
    """[(tensor, (min, max))] in order of first appearance."""
    ranges, order = parse_ranges(lines)
    out = []
    for name in order:
        mins, maxs = ranges[name]
        samples = len(mins)
        lo = float(np.percentile(mins, percentile))
        hi = float(np.percentile(maxs, 100 - percentile))
        if not lo < hi:
            raise ValueError("min should be < max, %s min:%f max:%f" % (name, lo, hi))
        if enhance and samples > 1:
            smin = np.sort(mins)
            smax = np.sort(maxs)[::-1]
            lo_idx = hi_idx = 0
            for i in range(samples):
                if smin[i] + 0.1 > hi:
                    break
                d_range = (smin[i] - lo) / (hi - lo)
                d_quant = float(i - lo_idx) / (samples - lo_idx)
                if d_quant > 0 and d_range / d_quant > enhance_ratio:
                    lo_idx, lo = i, float(smin[i])
                if lo + 0.1 > smax[i]:
                    break
                d_range = (hi - smax[i]) / (hi - lo)
                d_quant = float(i - hi_idx) / (samples - hi_idx)
                if d_quant > 0 and d_range / d_quant > enhance_ratio:
                    hi_idx, hi = i, float(smax[i])
        out.append((name, (lo, hi)))
    return out


def adjust_range(in_min, in_max, non_zero):
    """(scale, zero_point, adjusted_min, adjusted_max) of a uint8 tensor covering
    [in_min, in_max] and zero."""
    out_max = max(0.0, in_max)
    out_min = min(0.0, in_min)
    if non_zero:
        out_min = min(out_min, in_min - (out_max - in_min) / 254.0)
    scale = (out_max - out_min) / 255.0
    eps = 1e-6
    if out_min < -eps and out_max > eps:
        zero = -out_min / scale
        zero_int = int(round(zero))
        if abs(zero - zero_int) > eps and non_zero:
            zero_int = int(math.ceil(zero))
    elif out_min > -eps:
        zero_int = 0
    else:
        zero_int = 255
    return scale, zero_int, -zero_int * scale, (255 - zero_int) * scale
