"""Shared test utilities (CPU side)."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FORMATS = ((3, 2), (2, 2))                       # what the reference dispatches
ALL_FORMATS = FORMATS + ((2, 1), (3, 1), (2, 3))   # plus the other instantiations of its templates that this library takes
KAT_ONES_E3M2 = (806142768, 3274706115, 214118412)                          # reference tests/python/kernel_test_fpx.py:124-131
KAT_ONES_E2M2 = (272762913, 1107829124, 136414224, 562303042, 2215657992)   # reference tests/python/kernel_test_fpx.py:92-107


def kat_ones(e, m, rows, cols):
    """Unpacked weights whose every code is 1.0, built from the reference tests' known-answer words."""
    words = KAT_ONES_E3M2 if e == 3 else KAT_ONES_E2M2
    bw = 1 + e + m
    per_row = cols * bw // 32
    row = np.array([words[i % len(words)] for i in range(per_row)], dtype=np.uint32).astype(np.int32)
    return np.tile(row, (rows, 1))


def random_unpacked(rng, rows, cols, e, m):
    bw = 1 + e + m
    return rng.integers(-2**31, 2**31, size=(rows, cols * bw // 32), dtype=np.int64).astype(np.int32)


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))
