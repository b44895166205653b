"""Shared helpers of the parity tests."""

import numpy as np
import torch

# Tolerances of the acceptance contract: relative to the largest reference entry.
TOL_FP32 = 1e-5
TOL_HALF = 2e-2


def rel(got, want) -> float:
    """max|got - want| / max|want| with both sides taken to float64."""
    if isinstance(got, torch.Tensor):
        got = got.detach().double().cpu().numpy()
    if isinstance(want, torch.Tensor):
        want = want.detach().double().cpu().numpy()
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return 0.0
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def n64(x):
    return None if x is None else x.detach().double().cpu().numpy()


def tol(dtype) -> float:
    return TOL_FP32 if dtype == torch.float32 else TOL_HALF
