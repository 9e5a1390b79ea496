"""Seeded cases shared by the fixture generator's consumers: the same
(seed, shape) table as tests/golden/make_golden.py, rebuilt from the seed."""
from __future__ import annotations

import hashlib
import importlib.util
import os

import numpy as np

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

DECODE_CASES = make_golden.DECODE_CASES
LINEAR_CASES = make_golden.LINEAR_CASES
MOE_CASE = make_golden.MOE_CASE
linear_inputs = make_golden.linear_inputs
moe_inputs = make_golden.moe_inputs


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(a) -> np.ndarray:
    """Raw bit view for exact comparisons (float16 -> uint16, float32 -> uint32)."""
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def rel_err(got, want) -> float:
    """max |got - want| / max |want| -- the reference's GEMV tolerance measure
    (tests/test_metal.py:68-72 of the reference)."""
    g = np.asarray(got, dtype=np.float64)
    w = np.asarray(want, dtype=np.float64)
    return float(np.abs(g - w).max() / max(np.abs(w).max(), 1e-30))
