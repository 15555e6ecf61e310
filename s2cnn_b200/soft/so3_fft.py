"""SO(3) generalised FFTs and their autograd wrappers.

Same names, arguments and shapes as s2cnn/soft/so3_fft.py (so3_fft :12, so3_rfft :64, so3_ifft
:115, so3_rifft :158, SO3_fft_real :446, SO3_ifft_real :459).  The work is done by the CUDA
library; tensors must be float32 CUDA tensors.

Two deliberate differences, both invisible at the reference's own tolerances:

* ``so3_rifft`` returns the real part of the complex synthesis for any spectrum (the reference's
  CPU semantics); the reference's CUDA kernel assumed a Hermitian spectrum.
* ``SO3_fft_real.backward`` therefore uses the real-output synthesis directly instead of the
  complex one followed by ``[..., 0]`` (so3_fft.py:453-456) - same values, half the work.
"""
import torch

from ..ops import bandwidth_from_so3_nspec, cuda_ops


def so3_fft(x, for_grad=False, b_out=None):
    '''
    :param x: [..., beta, alpha, gamma, complex]
    :return: [l * m * n, ..., complex]
    '''
    return cuda_ops().so3_fft(x, for_grad=for_grad, b_out=b_out)


def so3_rfft(x, for_grad=False, b_out=None):
    '''
    :param x: [..., beta, alpha, gamma]
    :return: [l * m * n, ..., complex]
    '''
    return cuda_ops().so3_rfft(x, for_grad=for_grad, b_out=b_out)


def so3_ifft(x, for_grad=False, b_out=None):
    '''
    :param x: [l * m * n, ..., complex]
    :return: [..., beta, alpha, gamma, complex]
    '''
    return cuda_ops().so3_ifft(x, for_grad=for_grad, b_out=b_out)


def so3_rifft(x, for_grad=False, b_out=None):
    '''
    :param x: [l * m * n, ..., complex]
    :return: [..., beta, alpha, gamma]
    '''
    return cuda_ops().so3_rifft(x, for_grad=for_grad, b_out=b_out)


class SO3_fft_real(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, b_out=None):  # pylint: disable=W
        ctx.b_out = b_out
        ctx.b_in = x.size(-1) // 2
        return so3_rfft(x, b_out=ctx.b_out)

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        return so3_rifft(grad_output.contiguous(), for_grad=True, b_out=ctx.b_in), None


class SO3_fft_real_relu(torch.autograd.Function):
    """``SO3_fft_real`` of ``relu(x)`` with the activation applied while the signal is read (the
    ReLU between two convolutions of the reference's models, e.g. examples/mnist/run.py:88-93,
    folded into the consumer).  Needs 2 b_in <= 32."""

    @staticmethod
    def forward(ctx, x, b_out=None):  # pylint: disable=W
        ctx.b_in = x.size(-1) // 2
        ctx.save_for_backward(x)
        return cuda_ops().so3_rfft(x, b_out=b_out, relu=True)

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        (x,) = ctx.saved_tensors
        # the synthesis kernel writes 0 where x <= 0: no separate pass over the gradient signal
        return cuda_ops().so3_rifft_relu_grad(grad_output.contiguous(), x), None


class SO3_ifft_real(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, b_out=None):  # pylint: disable=W
        ctx.b_out = b_out
        ctx.b_in = bandwidth_from_so3_nspec(x.size(0))
        return so3_rifft(x, b_out=ctx.b_out)

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        return so3_rfft(grad_output.contiguous(), for_grad=True, b_out=ctx.b_in), None


class SO3_ifft_real_bias(torch.autograd.Function):
    """``SO3_ifft_real`` followed by ``+ bias`` ([1, f_out, 1, 1, 1]) in one pass: the addition
    of s2cnn/soft/s2_conv.py:45 and so3_conv.py:56 is fused into the last synthesis kernel."""

    @staticmethod
    def forward(ctx, x, bias):  # pylint: disable=W
        ctx.b_in = bandwidth_from_so3_nspec(x.size(0))
        ctx.bias_shape = bias.shape
        return cuda_ops().so3_rifft(x, bias=bias.reshape(-1))

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        grad_output = grad_output.contiguous()
        gx = gb = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and grad_output.dim() == 5:
            # the bias gradient is a by-product of the analysis kernel (per-signal sums)
            gx, sums = cuda_ops().so3_rfft_with_sums(grad_output, for_grad=True, b_out=ctx.b_in)
            return gx, sums.sum(dim=0).reshape(ctx.bias_shape)
        if ctx.needs_input_grad[0]:
            gx = so3_rfft(grad_output, for_grad=True, b_out=ctx.b_in)
        if ctx.needs_input_grad[1]:
            gb = grad_output.sum(dim=(0, 2, 3, 4)).reshape(ctx.bias_shape)
        return gx, gb
