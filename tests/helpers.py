"""Seeded problem generators shared by the CPU and GPU tests (kept in the package's harness so
that the benchmark and the smoke check can use them without the test tree)."""
from mace_b200.harness.cases import conv_quant, gemm_case, near_ratio  # noqa: F401
