"""The uniform variates behind the Gumbel noise must lie strictly inside (0, 1): u == 1 would give
-log(-log(1)) = +inf and that vocabulary entry would win the arg-max whatever its logit."""
import ctypes
import math

import numpy as np

from smcsd_b200.ops import native as K


def _fn():
    L = K.lib()
    L.smc_u32_to_unit.argtypes = [ctypes.c_uint]
    L.smc_u32_to_unit.restype = ctypes.c_float
    return L.smc_u32_to_unit


def test_u32_to_unit_is_open_interval():
    f = _fn()
    lo, hi = f(0), f(0xFFFFFFFF)
    assert 0.0 < lo < 1.0 and 0.0 < hi < 1.0
    for u in (lo, hi, f(0x80000000), f(0xFFFFFE00), f(0x1FF)):
        u32 = np.float32(u)
        g = -np.log(-np.log(u32, dtype=np.float32), dtype=np.float32)
        assert math.isfinite(float(g))


def test_u32_to_unit_is_monotone_and_exact():
    f = _fn()
    xs = [0, 1 << 9, 5 << 9, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF]
    vals = [f(x) for x in xs]
    assert all(a <= b for a, b in zip(vals, vals[1:]))
    for x, v in zip(xs, vals):
        assert v == ((x >> 9) + 0.5) / 8388608.0        # exactly representable, no rounding to 1.0
