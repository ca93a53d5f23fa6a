"""Shared by the parity tests: error measures of the reference's tests/verify.py:10-11."""
import numpy as np


def relative(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12))


def max_relative(a, b):
    """Largest elementwise error relative to the largest reference magnitude."""
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))
