"""The polynomial 2^x of ``csrc/kernels/packed_math.cuh`` (``ex2_poly2``), replayed in float32.

The attention backward computes half of its probabilities with it instead of the special-function
unit.  This test reads the coefficients out of the header, repeats the kernel's arithmetic
step by step in numpy float32 (round to nearest by the 1.5 * 2^23 addition, cubic on [-0.5, 0.5],
integer add into the exponent field) and checks the relative error over the range the kernels
use, the clamp at -126 and the exponent arithmetic for negative integers.
"""
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _coefficients():
    src = open(os.path.join(ROOT, "csrc", "kernels", "packed_math.cuh")).read()
    body = src[src.index("void ex2_poly2"):]
    body = body[:body.index("\n}\n")]
    c = [float(x) for x in re.findall(r"pack2\((-?[0-9.]+)f, \1f\)", body)]
    # order of appearance: -1 (for x - n), then c3, c2, c1, c0; the rounding constant is named
    assert len(c) == 5 and c[0] == -1.0, c
    assert "kMagic = 12582912.f" in body and "-126.f" in body
    return c[1:]


def _ex2_poly(x):
    c3, c2, c1, c0 = (np.float32(v) for v in _coefficients())
    magic = np.float32(12582912.0)
    x = np.maximum(x.astype(np.float32), np.float32(-126.0))
    t = (x + magic).astype(np.float32)
    n = (t - magic).astype(np.float32)
    f = (x - n).astype(np.float32)
    p = (c3 * f + c2).astype(np.float32)
    p = (p * f + c1).astype(np.float32)
    p = (p * f + c0).astype(np.float32)
    bits = (p.view(np.int32).astype(np.int64) + (t.view(np.int32).astype(np.int64) << 23)) & 0xFFFFFFFF
    return bits.astype(np.uint32).view(np.float32)


def test_relative_error_over_the_range_the_kernels_use():
    x = np.linspace(-126.0, 8.0, 400001).astype(np.float32)
    got = _ex2_poly(x).astype(np.float64)
    want = np.exp2(x.astype(np.float64))
    assert np.abs(got / want - 1.0).max() < 2e-4          # far below the 2^-9 of a bf16 result


def test_integers_halves_and_the_clamp():
    x = np.array([0.0, -1.0, -3.0, -17.0, 5.0, -0.5, 0.5, -126.0, -1e9, -np.inf], dtype=np.float32)
    got = _ex2_poly(x).astype(np.float64)
    want = np.exp2(np.maximum(x.astype(np.float64), -126.0))
    assert np.allclose(got, want, rtol=2e-4, atol=0.0)
    assert np.isfinite(got).all()
