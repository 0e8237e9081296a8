"""Module path of the reference's host-Adam builder (flextrain/ops/op_builder/cpu_adam.py:11-36).

The reference picks ``-D__AVX512__`` / ``-D__AVX256__`` / ``-D__SCALAR__`` from the CPU it
is built on; the host library here carries the AVX-512 and the scalar loop in one binary and
chooses at run time (``ft_adam_simd_width``).
"""
from . import CPUAdamBuilder

__all__ = ["CPUAdamBuilder"]
