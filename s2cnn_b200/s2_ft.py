"""s2_rft: transform of a kernel sampled on a few sphere points to its S2 spectrum.

Mirrors s2cnn/s2_ft.py:8-24.  The Fourier matrix F[i, (l,m)] = 2b conj(D^l_m0(alpha_i, beta_i, 0))
is generated in float64 by the library's host code (no lie_learn), cached per (b, grid, device)
like the reference's lru_cache (s2_ft.py:53-60); the product with the kernel and its transpose
(for autograd) run as CUDA kernels.
"""
from functools import lru_cache

import torch

from .ops import cuda_ops


class _Rft(torch.autograd.Function):
    """x2d [nf, n_grid] -> [nspec, nf, 2] with the Fourier matrix F [n_grid, nspec, 2]; ``Ft`` is
    the same matrix stored [nspec, 2, n_grid] (or None), the layout the tensor-core kernel wants
    for the forward product (both operands contiguous along the contraction)."""

    @staticmethod
    def forward(ctx, x2d, F, Ft=None):
        ctx.save_for_backward(F)
        if Ft is not None:
            return cuda_ops().rft_forward_t(x2d, Ft)
        return cuda_ops().rft_forward(x2d, F)

    @staticmethod
    def backward(ctx, g):
        (F,) = ctx.saved_tensors
        return cuda_ops().rft_backward(g.contiguous(), F), None, None


def fourier_matrices(F_host, device):
    """(F, Ft) on the device: Ft only for a CUDA device and an even number of grid points (the
    tensor-core product works on pairs along the contraction)."""
    F = torch.from_numpy(F_host).to(device)
    Ft = None
    if F.is_cuda and F.size(0) % 2 == 0:
        Ft = F.permute(1, 2, 0).contiguous()
    return F, Ft


@lru_cache(maxsize=32)
def _setup_s2_ft(b, grid, device_type, device_index):
    F = cuda_ops().s2_ft_matrix(b, grid)  # [n_grid, b^2, 2] float32, host
    return fourier_matrices(F, torch.device(device_type, device_index))


def s2_rft(x, b, grid):
    """
    Real Fourier Transform
    :param x: [..., beta_alpha]
    :param b: output bandwidth signal
    :param grid: tuple of (beta, alpha) tuples
    :return: [l * m, ..., complex]
    """
    F, Ft = _setup_s2_ft(b, grid, device_type=x.device.type, device_index=x.device.index)
    assert x.size(-1) == F.size(0)
    sz = x.size()
    out = _Rft.apply(x.reshape(-1, x.size(-1)), F, Ft)  # [l * m, prod(...), complex]
    return out.view(-1, *sz[:-1], 2)
