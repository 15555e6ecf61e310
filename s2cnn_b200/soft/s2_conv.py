"""S2Convolution (s2cnn/soft/s2_conv.py:13-47): same constructor, parameters, init and scaling."""
import math

import torch
from torch.nn.modules import Module
from torch.nn.parameter import Parameter

from ..ops import cuda_ops
from ..s2_ft import s2_rft
from .s2_fft import S2_fft_real
from .so3_fft import so3_rfft, SO3_fft_real, SO3_fft_real_relu
from ._spectrum_cache import KernelSpectrumCache
from ._recompute import fused_or_recompute


class _S2ProductSynthesis(torch.autograd.Function):
    """``SO3_ifft_real(s2_mm(x, y)) + bias`` (s2_conv.py:42-45) as one op: for small bandwidths the
    product is evaluated inside the synthesis kernel and the SO(3) spectrum never reaches memory.
    Backward is the reference's chain: so3_rfft(for_grad) of the output gradient, then the grad-x /
    grad-y products (s2cnn/soft/so3_fft.py:467-469, s2cnn/s2_mm.py:67-101)."""

    @staticmethod
    def forward(ctx, x, y, bias):  # pylint: disable=W
        ctx.save_for_backward(x, y)
        ctx.bias_shape = bias.shape
        return cuda_ops().s2_conv_synthesis(x, y, bias.reshape(-1))

    @staticmethod
    def backward(ctx, grad_output):  # pylint: disable=W
        x, y = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        gx = gy = gb = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            b = round(x.size(0) ** 0.5)
            if ctx.needs_input_grad[2] and grad_output.dim() == 5:
                # the bias gradient is a by-product of the analysis kernel (per-signal sums)
                gz, sums = cuda_ops().so3_rfft_with_sums(grad_output, for_grad=True, b_out=b)
                gb = sums.sum(dim=0).reshape(ctx.bias_shape)
            else:
                gz = so3_rfft(grad_output, for_grad=True, b_out=b)  # [l * m * n, batch, f_out, complex]
            if ctx.needs_input_grad[0]:
                gx = cuda_ops().s2_mm_gradx(gz, y, x.size(1), x.size(2))
            if ctx.needs_input_grad[1]:
                gy = cuda_ops().s2_mm_grady(gz, x, y.size(2))
        if ctx.needs_input_grad[2] and gb is None:
            gb = grad_output.sum(dim=(0, 2, 3, 4)).reshape(ctx.bias_shape)
        return gx, gy, gb


class S2Convolution(Module):
    def __init__(self, nfeature_in, nfeature_out, b_in, b_out, grid):
        """Correlation of a signal on the sphere with a learned kernel supported on a few points of
        the sphere; the result is a signal on SO(3).

        nfeature_in, nfeature_out: channel counts of the input and output signals.
        b_in, b_out: bandwidths; the input lives on the 2 b_in x 2 b_in sphere grid, the output on
            the (2 b_out)^3 SOFT grid.
        grid: the points (beta, alpha) on which the kernel has a weight, a tuple of 2-tuples;
            ``kernel`` holds one weight per (input channel, output channel, point).
        """
        super().__init__()
        self.nfeature_in = nfeature_in
        self.nfeature_out = nfeature_out
        self.b_in = b_in
        self.b_out = b_out
        self.grid = grid
        # one uniform_(-1, 1) draw on the default generator, as s2_conv.py:28
        self.kernel = Parameter(torch.empty(nfeature_in, nfeature_out, len(grid)).uniform_(-1, 1))
        self.scaling = 1. / math.sqrt(len(self.grid) * self.nfeature_in * (self.b_out ** 4.) / (self.b_in ** 2.))
        self.bias = Parameter(torch.zeros(1, nfeature_out, 1, 1, 1))
        self._spectrum_cache = KernelSpectrumCache()

    def forward(self, x, relu_so3_fft=None, channel_scale=None, bias=None):
        '''
        :x:      [batch, feature_in,  beta, alpha]
        :relu_so3_fft: (extension) bandwidth b_next of the SO3Convolution that follows: return
                 SO3_fft_real(relu(conv(x)), b_next) - that layer's input spectrum
                 [l * m * n, batch, feature_out, complex] (pass it on with ``input_spectrum=True``).
                 Without autograd and for 2 b_out <= 32 the signal between the layers is never written.
        :channel_scale, bias: (extension, used by ``s2cnn_b200.fuse`` to fold an eval-mode BatchNorm3d
                 into the layer) multiply output channel j by channel_scale[j] - applied to the
                 kernel's spectrum - and add ``bias`` ([1, f_out, 1, 1, 1]) instead of the layer's own
        :return: [batch, feature_out, beta, alpha, gamma]
        '''
        assert x.size(1) == self.nfeature_in
        assert x.size(2) == 2 * self.b_in
        assert x.size(3) == 2 * self.b_in
        x = S2_fft_real.apply(x, self.b_out)  # [l * m, batch, feature_in, complex]
        # [l * m, feature_in, feature_out, complex]; kept between calls while the weights stand still
        y = self._spectrum_cache.get(self.kernel, lambda k: s2_rft(k * self.scaling, self.b_out, self.grid))
        if channel_scale is not None:
            y = y * channel_scale.view(1, 1, -1, 1)
        own_bias = self.bias if bias is None else bias
        if relu_so3_fft is not None:
            b_next = int(relu_so3_fft)
            if 2 * self.b_out <= 32:   # ReLU applied while the next layer's analysis reads the signal
                plain = lambda xx, yy, bb: SO3_fft_real_relu.apply(_S2ProductSynthesis.apply(xx, yy, bb), b_next)  # noqa: E731
            else:
                plain = lambda xx, yy, bb: SO3_fft_real.apply(torch.relu(_S2ProductSynthesis.apply(xx, yy, bb)), b_next)  # noqa: E731
            if 2 * self.b_out <= 32 and b_next <= self.b_out:
                fused = lambda xx, yy, bb: cuda_ops().s2_conv_relu_so3_rfft(xx, yy, bb, b_next)  # noqa: E731
                grad = torch.is_grad_enabled() and (x.requires_grad or y.requires_grad or own_bias.requires_grad)
                return fused_or_recompute(fused, plain, (x, y, own_bias), grad,
                                          getattr(self, "fused_training", False))
            return plain(x, y, own_bias)
        # s2_mm -> SO3_ifft_real -> + bias, fused: [batch, feature_out, beta, alpha, gamma]
        return _S2ProductSynthesis.apply(x, y, own_bias)
