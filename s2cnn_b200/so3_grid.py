"""Sampling grids for SO(3) kernels: tuples of (beta, alpha, gamma) float triples.

Same point sets, order and arithmetic as the reference's s2cnn/so3_grid.py:6-54.
"""
import warnings

import numpy as np


def _triples(beta, alpha, gamma, shear=False):
    bb, aa, cc = np.meshgrid(beta, alpha, gamma, indexing="ij")
    if shear:
        cc = cc - aa  # gamma = pre_gamma - alpha (so3_grid.py:18)
    pts = tuple((float(b), float(a), float(c))
                for b, a, c in zip(bb.ravel(), aa.ravel(), cc.ravel()))
    if sum(1 for p in pts if p[0] == 0) > 1:
        warnings.warn("Gimbal lock: beta take value 0 in the grid")
    return pts


def _ring(n_alpha):
    return np.linspace(start=0, stop=2 * np.pi, num=n_alpha, endpoint=False)


def so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                           n_gamma=None):
    """Rings of rotations around the identity; size n_alpha * n_beta * n_gamma."""
    if n_gamma is None:
        n_gamma = n_alpha
    beta = np.arange(start=1, stop=n_beta + 1, dtype=float) * max_beta / n_beta
    pre_gamma = np.linspace(start=-max_gamma, stop=max_gamma, num=n_gamma, endpoint=True)
    return _triples(beta, _ring(n_alpha), pre_gamma, shear=True)


def so3_equatorial_grid(max_beta=0, max_gamma=np.pi / 8, n_alpha=32, n_beta=1, n_gamma=2):
    """Rings of rotations around the equator."""
    beta = np.linspace(start=np.pi / 2 - max_beta, stop=np.pi / 2 + max_beta, num=n_beta,
                       endpoint=True)
    gamma = np.linspace(start=-max_gamma, stop=max_gamma, num=n_gamma, endpoint=True)
    return _triples(beta, _ring(n_alpha), gamma)


def so3_soft_grid(b):
    beta = (np.arange(2 * b) + 0.5) / (2 * b) * np.pi
    ang = _ring(2 * b)
    return _triples(beta, ang, ang)
