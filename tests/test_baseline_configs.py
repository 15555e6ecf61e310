"""The reference's benchmark configurations at their real layer sizes (batch reduced so that the
CPU oracle finishes in seconds), on the GPU: outputs and - where the configuration trains - input,
weight and bias gradients against the oracle, within the stated tolerance (relative L2 <= 1e-4).

  config 0   S2Convolution 1 -> 20, b 30 -> 10, s2_near_identity_grid(pi/16, 8, 3)
  config 1   SO3Convolution 20 -> 40, b 10 -> 6, so3_near_identity_grid(pi/8, 2 pi, 8, 3, 8), fwd + bwd
  config 3   S2Conv -> ReLU -> SO3Conv -> ReLU -> so3_integrate -> Linear(40 -> 10), forward,
             with the activations fused the way bench.py runs the network
"""
import numpy as np
import pytest
import torch

from oracle import s2cnn_oracle as O
from util import assert_close

pytestmark = pytest.mark.gpu


def _grids():
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    return g2, g3


def _check_layer(conv, oracle_fn, x, b_in, b_out, grid, name):
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(7)
    with torch.no_grad():
        conv.bias.copy_(torch.randn(conv.bias.shape, generator=gen))
    k = conv.kernel.detach().clone().requires_grad_(True)
    bias = conv.bias.detach().clone().requires_grad_(True)
    xo = x.clone().requires_grad_(True)
    yo = oracle_fn(xo, k, bias, b_in, b_out, grid)
    gy = torch.randn(yo.shape, generator=gen)
    yo.backward(gy)

    conv = conv.to(dev)
    xd = x.clone().to(dev).requires_grad_(True)
    y = conv(xd)
    assert_close(y, yo.detach(), name + " y")
    y.backward(gy.to(dev))
    assert_close(xd.grad, xo.grad, name + " gx")
    assert_close(conv.kernel.grad, k.grad, name + " gkernel")
    assert_close(conv.bias.grad, bias.grad, name + " gbias")


def test_config0_s2_convolution_layer():
    import s2cnn_b200 as S
    g2, _ = _grids()
    torch.manual_seed(0)
    conv = S.S2Convolution(1, 20, 30, 10, g2)
    x = torch.randn(3, 1, 60, 60)
    _check_layer(conv, O.s2_convolution, x, 30, 10, g2, "config 0")


def test_config1_so3_convolution_layer_with_gradients():
    import s2cnn_b200 as S
    _, g3 = _grids()
    torch.manual_seed(1)
    conv = S.SO3Convolution(20, 40, 10, 6, g3)
    x = torch.randn(3, 20, 20, 20, 20)
    _check_layer(conv, O.so3_convolution, x, 10, 6, g3, "config 1")


def test_config3_network_forward_fused_activations():
    import s2cnn_b200 as S
    g2, g3 = _grids()
    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    c1 = S.S2Convolution(1, 20, 30, 10, g2)
    c2 = S.SO3Convolution(20, 40, 10, 6, g3)
    lin = torch.nn.Linear(40, 10)
    x = torch.randn(5, 1, 60, 60)
    with torch.no_grad():
        h = torch.relu(O.s2_convolution(x, c1.kernel, c1.bias, 30, 10, g2))
        h = torch.relu(O.so3_convolution(h, c2.kernel, c2.bias, 10, 6, g3))
        ref = lin(O.so3_integrate(h))
        c1, c2, lin = c1.to(dev), c2.to(dev), lin.to(dev)
        xd = x.to(dev)
        plain = lin(S.so3_integrate(torch.relu(c2(torch.relu(c1(xd))))))
        fused = lin(S.so3_relu_integrate(c2(c1(xd), relu_input=True)))
        tail = lin(c2(c1(xd), relu_input=True, relu_integrate=True))
        relay = lin(c2(c1(xd, relu_so3_fft=c2.b_out), input_spectrum=True, relu_integrate=True))
    assert_close(plain, ref, "config 3 logits, separate ReLUs")
    assert_close(fused, ref, "config 3 logits, ReLUs applied on load")
    assert_close(tail, ref, "config 3 logits, ReLU + integration inside the synthesis")
    assert_close(relay, ref, "config 3 logits, both layers' transforms in one kernel")
