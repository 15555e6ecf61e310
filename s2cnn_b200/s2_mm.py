"""s2_mm: per-degree product of an S2 signal spectrum with an S2 kernel spectrum.

Mirrors s2cnn/s2_mm.py:10-101 (function and autograd rule); all three products run in the
grouped complex GEMM kernel of the library.
"""
import torch

from .ops import cuda_ops


class _cuda_S2_mm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y):
        ctx.save_for_backward(x, y)
        return cuda_ops().s2_mm(x, y)

    @staticmethod
    def backward(ctx, gradz):
        x, y = ctx.saved_tensors
        gradz = gradz.contiguous()
        gradx = grady = None
        if ctx.needs_input_grad[0]:
            gradx = cuda_ops().s2_mm_gradx(gradz, y, x.size(1), x.size(2))
        if ctx.needs_input_grad[1]:
            grady = cuda_ops().s2_mm_grady(gradz, x, y.size(2))
        return gradx, grady


def s2_mm(x, y):
    '''
    :param x: [l * m,     batch,      feature_in,  complex]
    :param y: [l * m,     feature_in, feature_out, complex]
    :return:  [l * m * n, batch,      feature_out, complex]
    '''
    assert y.size(3) == 2
    assert x.size(3) == 2
    assert y.size(1) == x.size(2)
    assert y.size(0) == x.size(0)
    return _cuda_S2_mm.apply(x, y)
