"""The single-expression requantization used by the CUDA epilogues equals the two-step
gemmlowp definition (SRDHM, then rounding right shift) that the oracle implements.

Device formula (mace_b200/csrc/common.cuh, mb_requant_fast), modelled here with Python
integers:  y = (acc*mult + 2^30 + [s>=1]*2^(s+30) - [s>=1]*[acc<0]*2^31) >> (31 + s)
"""
import numpy as np


def device_formula(acc, mult, s):
    c64 = (1 << 30) + ((1 << (s + 30)) if s >= 1 else 0)
    neg = -(1 << 31) if s >= 1 else 0
    t = acc * mult + c64 + (1 if acc < 0 else 0) * neg
    assert -(1 << 63) <= t < (1 << 63)  # fits the 64-bit register pair
    return t >> (31 + s)


def test_identity_on_edges_ties_and_random_values(orc):
    rng = np.random.default_rng(0)
    edges = [0, 1, -1, 2, -2, 3, -3, 5, -5, 2 ** 31 - 1, -2 ** 31, 2 ** 30, -2 ** 30, 2 ** 30 + 1,
             -2 ** 30 - 1, 65025 * 4096, -65025 * 4096]
    mults = [2 ** 30, 2 ** 30 + 1, 2 ** 31 - 1, 1374221056, 1392511872]
    for s in range(0, 32):
        ms = mults + [int(m) for m in rng.integers(2 ** 30, 2 ** 31, size=3)]
        for m in ms:
            accs = edges + [int(a) for a in rng.integers(-2 ** 31, 2 ** 31, size=40)]
            accs += [int(a) for a in rng.integers(-70000, 70000, size=40)]
            # exact ties of the second stage: x = k * 2^s + 2^(s-1) needs acc ~ x * 2^31 / m
            for k in (-3, -1, 0, 1, 2):
                x = k * (1 << s) + ((1 << s) >> 1)
                a = (x << 31) // m
                accs += [a - 1, a, a + 1]
            for a in accs:
                if not (-2 ** 31 <= a < 2 ** 31):
                    continue
                assert device_formula(a, m, s) == orc.rounding_stages(a, m, s), (a, m, s)


def test_identity_exhaustive_small_range(orc):
    for s in (0, 1, 2, 3, 7):
        for m in (2 ** 30, 3 * 2 ** 29, 2 ** 31 - 1):
            for a in range(-3000, 3001):
                assert device_formula(a, m, s) == orc.rounding_stages(a, m, s), (a, m, s)


def device_formula_variants(acc, mult, s, zp0):
    """mb_requant_t of common.cuh: for s >= 1 the high word of t, shifted by s - 1; with an
    output zero point of 0 the [acc < 0] term is dropped."""
    c64 = (1 << 30) + ((1 << (s + 30)) if s >= 1 else 0)
    t = acc * mult + c64
    if s >= 1 and not zp0 and acc < 0:
        t -= 1 << 31
    assert -(1 << 63) <= t < (1 << 63)
    return ((t >> 32) >> (s - 1)) if s >= 1 else (t >> 31)


def test_variants_match_two_step_definition(orc):
    rng = np.random.default_rng(1)
    for s in range(0, 32):
        ms = [2 ** 30, 2 ** 30 + 1, 2 ** 31 - 1, 1374221056, 1392511872]
        ms += [int(m) for m in rng.integers(2 ** 30, 2 ** 31, size=3)]
        for m in ms:
            accs = [0, 1, -1, 2, -2, 3, -3, 2 ** 31 - 1, -2 ** 31]
            accs += [int(a) for a in rng.integers(-2 ** 31, 2 ** 31, size=60)]
            accs += [int(a) for a in rng.integers(-70000, 70000, size=60)]
            for k in (-3, -1, 0, 1, 2):
                x = k * (1 << s) + ((1 << s) >> 1)
                a = (x << 31) // m
                accs += [a - 1, a, a + 1]
            for a in accs:
                if not (-2 ** 31 <= a < 2 ** 31):
                    continue
                ref = orc.rounding_stages(a, m, s)
                assert device_formula_variants(a, m, s, False) == ref, (a, m, s)
                z = device_formula_variants(a, m, s, True)
                assert min(255, max(0, z)) == min(255, max(0, ref)), (a, m, s)


def device_formula_packed(acc, mult, s, zp):
    """mb_requant_pack4 of common.cuh (1 <= s <= 19): the output zero point rides in the rounding
    constant, the saturation to [0, 255] is done by the packing instruction."""
    assert 1 <= s <= 19 and 0 <= zp <= 255
    sh = 31 + s
    t = acc * mult + (1 << 30) + (1 << (s + 30)) + (zp << sh)
    if zp != 0 and acc < 0:  # the zero-point-0 variant drops the sign term
        t -= 1 << 31
    assert -(1 << 63) <= t < (1 << 63)
    y = (t >> 32) >> (sh - 32)
    assert -(1 << 31) <= y < (1 << 31)
    return min(255, max(0, y))


def test_packed_form_matches_two_step_definition(orc):
    rng = np.random.default_rng(2)
    for s in range(1, 20):
        ms = [2 ** 30, 2 ** 30 + 1, 2 ** 31 - 1, 1374221056] + [int(m) for m in rng.integers(2 ** 30, 2 ** 31, size=3)]
        for m in ms:
            accs = [0, 1, -1, 2, -2, 2 ** 31 - 1, -2 ** 31]
            accs += [int(a) for a in rng.integers(-2 ** 31, 2 ** 31, size=40)]
            accs += [int(a) for a in rng.integers(-300 * (1 << s), 300 * (1 << s), size=60)]
            for k in (-3, -1, 0, 1, 2, 254, 255):
                x = k * (1 << s) + ((1 << s) >> 1)
                a = (x << 31) // m
                accs += [a - 1, a, a + 1]
            for a in accs:
                if not (-2 ** 31 <= a < 2 ** 31):
                    continue
                ref = orc.rounding_stages(a, m, s)
                for zp in (0, 1, 77, 128, 255):
                    assert device_formula_packed(a, m, s, zp) == min(255, max(0, ref + zp)), (a, m, s, zp)
