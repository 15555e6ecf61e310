"""so3_rotation: rotate a signal on SO(3) through its spectrum (s2cnn/soft/so3_rotation.py:11-73).

analysis (SO3_fft_real) -> one grouped complex product with the block-diagonal Wigner-D matrices
of the rotation -> synthesis (SO3_ifft_real); all three steps are CUDA kernels of this library.
"""
from functools import lru_cache

import torch

from ..ops import cuda_ops
from .so3_fft import SO3_fft_real, SO3_ifft_real


@lru_cache(maxsize=32)
def _setup_so3_rotation(b, alpha, beta, gamma, device_type, device_index):
    """Concatenated U^l[m, n] = exp(i m alpha) d^l_mn(beta) exp(i n gamma), l < b, on the device.

    The reference builds these with lie_learn and caches them on disk and in an lru_cache
    (s2cnn/soft/so3_rotation.py:51-73); here the library's host recurrence produces them.
    """
    U = cuda_ops().so3_rotation_matrices(b, alpha, beta, gamma)
    return torch.from_numpy(U).to(torch.device(device_type, device_index))


class _RotateSpectrum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, U, b):
        ctx.b = b
        ctx.save_for_backward(U)
        return cuda_ops().so3_rotate_spectrum(U, x, b, adjoint=False)

    @staticmethod
    def backward(ctx, g):
        (U,) = ctx.saved_tensors
        return cuda_ops().so3_rotate_spectrum(U, g.contiguous(), ctx.b, adjoint=True), None, None


def so3_rotation(x, alpha, beta, gamma):
    """
    :param x: [..., beta, alpha, gamma] (..., 2b, 2b, 2b)
    """
    b = x.size()[-1] // 2
    x_size = x.size()
    U = _setup_so3_rotation(b, float(alpha), float(beta), float(gamma),
                            device_type=x.device.type, device_index=x.device.index)
    x = SO3_fft_real.apply(x)          # [l * m * n, ..., complex]
    z = _RotateSpectrum.apply(x, U, b)
    z = SO3_ifft_real.apply(z)
    return z.contiguous().view(*x_size)
