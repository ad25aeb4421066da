"""Shared test helpers: the reference's closeness rule and fixture loading."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "optimizer_vectors.json")


def load_golden():
    with open(GOLDEN, "r", encoding="utf-8") as f:
        return json.load(f)


def assert_close(name, got, want, atol, rtol):
    """|got - want| <= atol + rtol*|want|; NaN/Inf fail (autograd/test_helpers_test.go:12-23)."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    assert got.shape == want.shape, f"{name}: length {got.size} != {want.size}"
    assert np.all(np.isfinite(got)), f"{name}: non-finite value"
    diff = np.abs(got - want)
    bad = diff > atol + rtol * np.abs(want)
    if bad.any():
        i = int(np.argmax(bad))
        raise AssertionError(f"{name}[{i}]={got[i]:.9g} want {want[i]:.9g} (diff {diff[i]:.3g})")


def ulp_distance(a, b):
    """Distance in units in the last place between two float32 arrays (same sign region safe)."""
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7FFFFFFF), a)
    b = np.where(b < 0, -(b & 0x7FFFFFFF), b)
    return np.abs(a - b)


def f32(values):
    return np.array(values, dtype=np.float32)
