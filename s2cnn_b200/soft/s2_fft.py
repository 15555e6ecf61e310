"""S2 generalised FFTs and their autograd wrappers.

Same names, arguments and shapes as s2cnn/soft/s2_fft.py (s2_fft :13, s2_ifft :61, S2_fft_real
:226, S2_ifft_real :239).  ``S2_fft_real`` feeds the real signal straight to the kernel instead of
first materialising a complex copy (the reference's as_complex at :232).
"""
import torch

from ..ops import cuda_ops


def s2_fft(x, for_grad=False, b_out=None):
    '''
    :param x: [..., beta, alpha, complex]
    :return:  [l * m, ..., complex]
    '''
    return cuda_ops().s2_fft(x, for_grad=for_grad, b_out=b_out)


def s2_ifft(x, for_grad=False, b_out=None):
    '''
    :param x: [l * m, ..., complex]
    :return: [..., beta, alpha, complex]
    '''
    return cuda_ops().s2_ifft(x, for_grad=for_grad, b_out=b_out)


class S2_fft_real(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, b_out=None):  # pylint: disable=W
        ctx.b_out = b_out
        ctx.b_in = x.size(-1) // 2
        return cuda_ops().s2_fft(x, b_out=ctx.b_out, x_is_real=True)

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        return cuda_ops().s2_ifft(grad_output.contiguous(), for_grad=True, b_out=ctx.b_in,
                                  out_is_real=True), None


class S2_ifft_real(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, b_out=None):  # pylint: disable=W
        nspec = x.size(0)
        ctx.b_out = b_out
        ctx.b_in = round(nspec ** 0.5)
        return cuda_ops().s2_ifft(x, b_out=ctx.b_out, out_is_real=True)

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        return cuda_ops().s2_fft(grad_output.contiguous(), for_grad=True, b_out=ctx.b_in,
                                 x_is_real=True), None
