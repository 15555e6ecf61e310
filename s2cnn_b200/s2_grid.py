"""Sampling grids for S2 kernels: tuples of (beta, alpha) float pairs (hashable, float64).

Same point sets, order and arithmetic as the reference's s2cnn/s2_grid.py:5-40, so that the
Fourier matrices built from them are identical.
"""
import numpy as np


def _pairs(beta, alpha):
    bb, aa = np.meshgrid(beta, alpha, indexing="ij")
    return tuple((float(b), float(a)) for b, a in zip(bb.ravel(), aa.ravel()))


def _ring(n_alpha):
    return np.linspace(start=0, stop=2 * np.pi, num=n_alpha, endpoint=False)


def s2_near_identity_grid(max_beta=np.pi / 8, n_alpha=8, n_beta=3):
    """n_beta rings around the north pole, n_alpha points each (beta-major order)."""
    beta = np.arange(start=1, stop=n_beta + 1, dtype=float) * max_beta / n_beta
    return _pairs(beta, _ring(n_alpha))


def s2_equatorial_grid(max_beta=0, n_alpha=32, n_beta=1):
    """n_beta rings around the equator."""
    beta = np.linspace(start=np.pi / 2 - max_beta, stop=np.pi / 2 + max_beta, num=n_beta,
                       endpoint=True)
    return _pairs(beta, _ring(n_alpha))


def s2_soft_grid(b):
    """The full SOFT sampling grid of bandwidth b."""
    beta = (np.arange(2 * b) + 0.5) / (2 * b) * np.pi
    return _pairs(beta, _ring(2 * b))
