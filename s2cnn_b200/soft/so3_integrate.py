"""so3_integrate: Haar integral of a signal on SO(3) (s2cnn/soft/so3_integrate.py:7-29)."""
import torch

from ..ops import cuda_ops


class _SO3Integrate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, relu):
        ctx.b = x.size(-1) // 2
        ctx.relu = relu
        if relu:
            ctx.save_for_backward(x)
        return cuda_ops().so3_integrate(x, relu=relu)

    @staticmethod
    def backward(ctx, g):
        x = ctx.saved_tensors[0] if ctx.relu else None
        return cuda_ops().so3_integrate_backward(g.contiguous(), ctx.b, x=x, relu=ctx.relu), None


def so3_integrate(x):
    """
    Integrate a signal on SO(3) using the Haar measure

    :param x: [..., beta, alpha, gamma] (..., 2b, 2b, 2b)
    :return y: [...] (...)
    """
    assert x.size(-1) == x.size(-2)
    assert x.size(-2) == x.size(-3)
    return _SO3Integrate.apply(x, False)


def so3_relu_integrate(x):
    """``so3_integrate(relu(x))`` in one pass over x (the activation is applied while reading)."""
    assert x.size(-1) == x.size(-2)
    assert x.size(-2) == x.size(-3)
    return _SO3Integrate.apply(x, True)
