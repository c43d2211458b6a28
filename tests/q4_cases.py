"""Shared helpers of the GPU parity tests."""
import numpy as np

TOLERANCE = 2e-3  # max|y - ref| / max|ref| with fp32 accumulation: the bound this library is built to


def relative_error(y, ref64):
    ref = np.asarray(ref64, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref)) / np.max(np.abs(ref)))


def assert_close(y, ref64, what=""):
    error = relative_error(y, ref64)
    assert np.isfinite(error) and error <= TOLERANCE, f"{what}: max|d|/max|ref| = {error:.3e}"
    return error


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    width = {2: np.uint16, 4: np.uint32, 1: np.uint8}[a.dtype.itemsize]
    return bool((a.view(width) == b.view(width)).all())
