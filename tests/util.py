"""Shared helpers for the test-suite: fixture loading and the error metrics.

Tolerances (float32 path):
* ``REL_L2_TOL = 1e-4``  - relative L2 error per output / gradient tensor (the stated bar).
* ``MAXSTD_TOL = 1e-4``  - the reference's own CPU-vs-GPU criterion ``max|d| / std(ref)``
  (tests/so3_fft.py:95-100, s2cnn/so3_mm.py:268-271).
"""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REL_L2_TOL = 1e-4
MAXSTD_TOL = 1e-4


def golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: (torch.from_numpy(z[k]) if z[k].dtype.kind == "f" and z[k].ndim > 0
                    else z[k]) for k in z.files}


def rel_l2(a, b):
    a = torch.as_tensor(a, dtype=torch.float64).cpu()
    b = torch.as_tensor(b, dtype=torch.float64).cpu()
    den = b.norm().item()
    return (a - b).norm().item() / (den if den > 0 else 1.0)


def max_over_std(a, b):
    a = torch.as_tensor(a, dtype=torch.float64).cpu()
    b = torch.as_tensor(b, dtype=torch.float64).cpu()
    s = b.std().item() if b.numel() > 1 else abs(b.item())
    return (a - b).abs().max().item() / (s if s > 0 else 1.0)


def assert_close(a, b, what=""):
    assert tuple(a.shape) == tuple(b.shape), (what, a.shape, b.shape)
    r = rel_l2(a, b)
    q = max_over_std(a, b)
    assert r <= REL_L2_TOL, "%s rel-L2 %.3e > %g" % (what, r, REL_L2_TOL)
    assert q <= MAXSTD_TOL, "%s max/std %.3e > %g" % (what, q, MAXSTD_TOL)


def grid_tuple(arr):
    return tuple(tuple(float(v) for v in row) for row in np.asarray(arr))
