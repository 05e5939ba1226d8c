"""Helpers shared by the GPU parity tests."""
import numpy as np

import arcint_b200 as A
import oracle as O


def rel_err(got, ref):
    """max relative error against max(|ref|, 1e-2 * max|ref| of the column)"""
    ref = np.asarray(ref, dtype=np.float64)
    floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
    floor = np.maximum(floor, 1e-30)
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), floor)).max())


def nmse(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(((got - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-300))


TOL = 1e-3          # max relative error against the fp64 product of the same quantized operands


def make_weights(t, m, k, seed, standin=True):
    """N(0, 0.02) weights quantized to type t (ggml rule for Q4_0/Q8_0, stand-in for the rest)."""
    return O.quantize(t, O.fill_normal(m * k, seed, 0.02).reshape(m, k))
