"""Shared helpers of the parity tests."""
import numpy as np

# Error measure of every parity test: the largest absolute deviation divided by
# the largest magnitude of the reference tensor (for logits: per sample, divided
# by that sample's largest |logit|).  An element-wise ratio is meaningless for
# the near-zero outputs a sum of mixed-sign products produces; normalising by the
# tensor's scale is the usual way to state GEMM accuracy.
# Tolerances of ONE contraction against the fp32 CPU oracle: TF32 products with
# fp32 accumulation 1e-3; the fp32 CUDA-core path and 3xTF32 1e-5.  (The tensor
# core's fp32 accumulator rounds toward zero on every K=8 step, a bias of about
# K * 7.5e-9; the 3xTF32 kernel therefore promotes partial sums to registers
# every 128 K elements.)
TOL = {"fp32": 1e-5, "tf32x3": 1e-5, "tf32": 1e-3}
# Whole networks: rounding compounds with depth.  Measured on the benchmark
# geometries: TF32 0.6-1.3e-3 (operand rounding 2^-11 per layer, growing about
# sqrt(layers)), 3xTF32 0.4-2.6e-5.
NET_TOL = {"fp32": 1e-5, "tf32x3": 5e-5, "tf32": 3e-3}


def rel_err(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def logit_err(a, b, rows):
    """Per-sample error: max_i |a_i - b_i| / max_i |b_i| for each row, worst row."""
    a = np.asarray(a, np.float64).reshape(rows, -1)
    b = np.asarray(b, np.float64).reshape(rows, -1)
    return float((np.abs(a - b).max(1) / (np.abs(b).max(1) + 1e-30)).max())


def elementwise_err(a, b, floor=0.05):
    """Informational: element-wise relative error with magnitudes below floor*max clamped."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    scale = np.maximum(np.abs(b), floor * np.abs(b).max() + 1e-30)
    return float((np.abs(a - b) / scale).max())


def assert_close(a, b, mode, what="", factor=1.0, rows=None, tol=None):
    assert np.isfinite(np.asarray(a)).all(), f"{what}: non-finite values in the result"
    e = rel_err(a, b) if rows is None else logit_err(a, b, rows)
    limit = (tol or TOL)[mode] * factor
    assert e <= limit, f"{what}: rel err {e:.3e} > {limit:.1e} in mode {mode}"
    return e
