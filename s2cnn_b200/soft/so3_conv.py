"""SO3Convolution and SO3Shortcut (s2cnn/soft/so3_conv.py:12-85): same constructors, parameters,
init, scaling and state_dict keys."""
import math

import torch
from torch.nn.modules import Module
from torch.nn.parameter import Parameter

from ..ops import cuda_ops
from ..so3_ft import so3_rft
from ..so3_mm import so3_mm
from .so3_fft import SO3_fft_real, SO3_fft_real_relu, SO3_ifft_real_bias
from .so3_integrate import so3_relu_integrate
from ._spectrum_cache import KernelSpectrumCache
from ._recompute import fused_or_recompute


class SO3Convolution(Module):
    def __init__(self, nfeature_in, nfeature_out, b_in, b_out, grid):
        """Correlation of an SO(3) signal with a learned kernel supported on a few group elements.

        nfeature_in, nfeature_out: channel counts of the input and output signals.
        b_in, b_out: bandwidths; the input lives on the (2 b_in)^3 SOFT grid, the output on the
            (2 b_out)^3 one.
        grid: the rotations (beta, alpha, gamma) on which the kernel has a weight, a tuple of
            3-tuples; ``kernel`` holds one weight per (input channel, output channel, rotation).
        """
        super().__init__()
        self.nfeature_in = nfeature_in
        self.nfeature_out = nfeature_out
        self.b_in = b_in
        self.b_out = b_out
        self.grid = grid
        self.kernel = Parameter(torch.empty(nfeature_in, nfeature_out, len(grid)).uniform_(-1, 1))
        self.bias = Parameter(torch.zeros(1, nfeature_out, 1, 1, 1))
        # the scaling stays outside the parameter (so3_conv.py:30-34)
        self.scaling = 1. / math.sqrt(len(self.grid) * self.nfeature_in * (self.b_out ** 3.) / (self.b_in ** 3.))
        self._spectrum_cache = KernelSpectrumCache()

    def forward(self, x, relu_input=False, relu_integrate=False, input_spectrum=False,
                relu_so3_fft=None, channel_scale=None, bias=None):
        '''
        :x:      [batch, feature_in,  beta, alpha, gamma]
        :input_spectrum: (extension) x is already SO3_fft_real(signal, b_out), as returned by
                         ``S2Convolution.forward(..., relu_so3_fft=b_out)``
        :relu_so3_fft: (extension) bandwidth b_next of the SO3Convolution that follows: return that
                       layer's input spectrum SO3_fft_real(relu(conv(x)), b_next) (see S2Convolution)
        :relu_input: (extension) compute conv(relu(x)); the activation is applied while x is read
        :relu_integrate: (extension) return so3_integrate(relu(conv(x))) [batch, feature_out]; without
                         autograd and for 2 b_out <= 32 the output signal is never written
        :channel_scale, bias: (extension, used by ``s2cnn_b200.fuse`` to fold an eval-mode BatchNorm3d
                         into the layer) multiply output channel j by channel_scale[j] - applied to
                         the kernel's spectrum, the layer being linear in it - and add ``bias``
                         ([1, f_out, 1, 1, 1]) instead of the layer's own
        :return: [batch, feature_out, beta, alpha, gamma]
        '''
        if input_spectrum:
            assert x.dim() == 4 and x.size(2) == self.nfeature_in and x.size(3) == 2
        else:
            assert x.size(1) == self.nfeature_in
            assert x.size(2) == 2 * self.b_in
            assert x.size(3) == 2 * self.b_in
            assert x.size(4) == 2 * self.b_in
            if relu_input and 2 * self.b_in <= 32:
                x = SO3_fft_real_relu.apply(x, self.b_out)
            else:
                if relu_input:
                    x = torch.relu(x)
                x = SO3_fft_real.apply(x, self.b_out)  # [l * m * n, batch, feature_in, complex]
        # [l * m * n, feature_in, feature_out, complex]; kept between calls while the weights stand still
        y = self._spectrum_cache.get(self.kernel, lambda k: so3_rft(k * self.scaling, self.b_out, self.grid))
        if channel_scale is not None:
            y = y * channel_scale.view(1, 1, -1, 1)
        own_bias = self.bias if bias is None else bias
        assert x.size(0) == y.size(0)
        assert x.size(2) == y.size(1)
        z = so3_mm(x, y)  # [l * m * n, batch, feature_out, complex]
        needs_grad = torch.is_grad_enabled() and (z.requires_grad or own_bias.requires_grad)
        opt_in = getattr(self, "fused_training", False)
        if relu_so3_fft is not None:
            b_next = int(relu_so3_fft)
            if 2 * self.b_out <= 32:   # ReLU applied while the next layer's analysis reads the signal
                plain = lambda zz, bb: SO3_fft_real_relu.apply(SO3_ifft_real_bias.apply(zz, bb), b_next)  # noqa: E731
            else:
                plain = lambda zz, bb: SO3_fft_real.apply(torch.relu(SO3_ifft_real_bias.apply(zz, bb)), b_next)  # noqa: E731
            if 2 * self.b_out <= 32 and b_next <= self.b_out:
                fused = lambda zz, bb: cuda_ops().so3_rifft_relu_rfft(zz, bb, self.b_out, b_next)  # noqa: E731
                return fused_or_recompute(fused, plain, (z, own_bias), needs_grad, opt_in)
            return plain(z, own_bias)
        if relu_integrate:
            plain = lambda zz, bb: so3_relu_integrate(SO3_ifft_real_bias.apply(zz, bb))  # noqa: E731
            if 2 * self.b_out <= 32:
                fused = lambda zz, bb: cuda_ops().so3_rifft_relu_integrate(zz, bias=bb)  # noqa: E731
                return fused_or_recompute(fused, plain, (z, own_bias), needs_grad, opt_in)  # [batch, feature_out]
            return plain(z, own_bias)
        return SO3_ifft_real_bias.apply(z, own_bias)  # [batch, feature_out, beta, alpha, gamma]


class SO3Shortcut(Module):
    """Skip connection for residual blocks: the identity when channel count and bandwidth are
    unchanged, otherwise an SO3Convolution whose kernel sits on the identity rotation alone (a
    per-channel mixing plus band limitation).  Parameters appear under ``conv.`` in the state dict
    as in the reference (so3_conv.py:61-85)."""

    def __init__(self, nfeature_in, nfeature_out, b_in, b_out):
        super().__init__()
        assert b_out <= b_in
        if (nfeature_in != nfeature_out) or (b_in != b_out):
            self.conv = SO3Convolution(
                nfeature_in=nfeature_in, nfeature_out=nfeature_out, b_in=b_in, b_out=b_out,
                grid=((0, 0, 0), ))
        else:
            self.conv = None

    def forward(self, x):
        """[batch, feature_in, 2 b_in, 2 b_in, 2 b_in] -> [batch, feature_out, 2 b_out, 2 b_out, 2 b_out]"""
        if self.conv is not None:
            return self.conv(x)
        return x
