"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda").contiguous()


def cosine(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-300))


def assert_close_attn(got, ref, max_abs=2e-2, cos=0.9995, what=""):
    """The output tolerance of the path: max-abs <= 2e-2 and cosine >= 0.9995 against the fp64 oracle."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.abs(got - ref).max()
    c = cosine(got, ref)
    assert err <= max_abs and c >= cos, "%s: max-abs %.3e (limit %.1e), cosine %.6f (limit %.4f)" % (what, err, max_abs, c, cos)
    return err, c
