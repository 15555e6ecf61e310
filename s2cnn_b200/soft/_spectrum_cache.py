"""Per-module cache of the kernel's spectrum.

``S2Convolution`` / ``SO3Convolution`` transform ``kernel * scaling`` to the spectral domain in
every forward pass (s2cnn/soft/s2_conv.py:41, so3_conv.py:47).  The result depends on the weights
alone, so in inference it is the same tensor pass after pass; the cache keeps it while the
parameter has not been written to (its version counter, storage and device are unchanged) and no
gradient with respect to it is being recorded.  During training the transform runs every time, as
autograd needs it in the graph.
"""
import torch


class KernelSpectrumCache:
    def __init__(self):
        self._key = None
        self._value = None

    def get(self, kernel, transform):
        if torch.is_grad_enabled() and kernel.requires_grad:
            return transform(kernel)
        key = (kernel._version, kernel.data_ptr(), kernel.device, tuple(kernel.shape))
        if self._key != key:
            with torch.no_grad():
                self._value = transform(kernel)
            self._key = key
        return self._value

    def clear(self):
        self._key = None
        self._value = None
