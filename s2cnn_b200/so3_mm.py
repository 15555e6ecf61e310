"""so3_mm: per-degree block product of an SO(3) signal spectrum with a kernel spectrum.

Mirrors s2cnn/so3_mm.py:8-122 (function and autograd rule).
"""
import torch

from .ops import bandwidth_from_so3_nspec, cuda_ops


class _cuda_SO3_mm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y):
        ctx.save_for_backward(x, y)
        return cuda_ops().so3_mm(x, y)

    @staticmethod
    def backward(ctx, gradz):
        x, y = ctx.saved_tensors
        gradz = gradz.contiguous()
        gradx = grady = None
        if ctx.needs_input_grad[0]:
            gradx = cuda_ops().so3_mm_gradx(gradz, y, x.size(1), x.size(2))
        if ctx.needs_input_grad[1]:
            grady = cuda_ops().so3_mm_grady(gradz, x, y.size(2))
        return gradx, grady


def so3_mm(x, y):
    '''
    :param x: [l * m * n,   batch,    feature_in,  complex]
    :param y: [l * m * n, feature_in, feature_out, complex]
    :return:  [l * m * n,   batch,    feature_out, complex]
    '''
    assert y.size(3) == 2
    assert x.size(3) == 2
    assert y.size(1) == x.size(2)
    assert y.size(0) == x.size(0)
    bandwidth_from_so3_nspec(x.size(0))  # asserts a valid spectrum length
    return _cuda_SO3_mm.apply(x, y)
