"""The reference-named public API (functions, autograd rules, nn.Modules) against golden vectors
produced by the reference's own modules (outputs and gradients), on both builds."""
import numpy as np
import pytest
import torch

import backends
from oracle import s2cnn_oracle as O
from util import assert_close, golden, grid_tuple


def _layer_case(backend, name, cls):
    import s2cnn_b200
    g = golden(name)
    with backends.active(backend) as (_, dev):
        grid = grid_tuple(g["grid"])
        f_in, f_out = g["kernel"].shape[:2]
        conv = getattr(s2cnn_b200, cls)(f_in, f_out, int(g["b_in"]), int(g["b_out"]), grid)
        with torch.no_grad():
            conv.kernel.copy_(g["kernel"])
            conv.bias.copy_(g["bias"])
        conv = conv.to(dev)
        x = g["x"].to(dev).requires_grad_(True)
        y = conv(x)
        assert_close(y, g["y"], name + " y")
        y.backward(g["gy"].to(dev))
        assert_close(x.grad, g["gx"], name + " gx")
        assert_close(conv.kernel.grad, g["gkernel"], name + " gkernel")
        assert_close(conv.bias.grad, g["gbias"], name + " gbias")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_s2_convolution(backend):
    _layer_case(backend, "s2_conv_6_4", "S2Convolution")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_so3_convolution(backend):
    _layer_case(backend, "so3_conv_5_3", "SO3Convolution")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_so3_shortcut(backend):
    import s2cnn_b200
    g = golden("so3_shortcut_4_3")
    with backends.active(backend) as (_, dev):
        sc = s2cnn_b200.SO3Shortcut(2, 4, 4, 3)
        assert set(sc.state_dict()) == {"conv.kernel", "conv.bias"}  # so3_conv.py:71
        with torch.no_grad():
            sc.conv.kernel.copy_(g["kernel"])
            sc.conv.bias.copy_(g["bias"])
        sc = sc.to(dev)
        assert_close(sc(g["x"].to(dev)), g["y"], "shortcut")
        ident = s2cnn_b200.SO3Shortcut(3, 3, 4, 4)
        assert ident.conv is None
        x = g["x"].to(dev)
        assert ident(x) is x
        with pytest.raises(AssertionError):
            s2cnn_b200.SO3Shortcut(2, 2, 3, 4)  # b_out > b_in (so3_conv.py:68)


def test_module_init_matches_reference_draw():
    """Same seed => same kernel draw as the reference's constructor (one uniform_(-1, 1) on the
    default CPU generator, s2cnn/soft/s2_conv.py:28), bias zero, same scaling."""
    import s2cnn_b200
    grid = s2cnn_b200.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    torch.manual_seed(7)
    conv = s2cnn_b200.S2Convolution(2, 3, 6, 4, grid)
    g = golden("s2_conv_6_4")
    assert torch.equal(conv.kernel.detach(), g["kernel"])
    assert conv.bias.abs().sum().item() == 0
    assert abs(conv.scaling - O.s2_conv_scaling(2, 6, 4, len(grid))) < 1e-15
    so3g = s2cnn_b200.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8,
                                             n_beta=3, n_gamma=8)
    conv3 = s2cnn_b200.SO3Convolution(2, 3, 5, 3, so3g)
    assert abs(conv3.scaling - O.so3_conv_scaling(2, 5, 3, len(so3g))) < 1e-15
    assert set(conv3.state_dict()) == {"kernel", "bias"}


def test_grids_bit_identical_to_reference():
    import s2cnn_b200 as S
    g = golden("grids")
    mine = {
        "s2_near": S.s2_near_identity_grid(),
        "s2_near_c0": S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3),
        "s2_eq": S.s2_equatorial_grid(max_beta=0.2, n_alpha=6, n_beta=3),
        "s2_soft": S.s2_soft_grid(3),
        "so3_near": S.so3_near_identity_grid(),
        "so3_near_c1": S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8,
                                                n_beta=3, n_gamma=8),
        "so3_eq": S.so3_equatorial_grid(max_beta=0.1, max_gamma=0.3, n_alpha=5, n_beta=2, n_gamma=3),
        "so3_soft": S.so3_soft_grid(2),
    }
    for k, v in mine.items():
        ref = g[k].numpy() if hasattr(g[k], "numpy") else g[k]
        assert np.array_equal(np.array(v), ref), k
        hash(v)  # grids must be hashable (they key the Fourier-matrix cache)


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_functional_api_names_and_autograd(backend):
    """s2_rft / so3_rft / s2_mm / so3_mm / so3_integrate / *_fft_real through autograd."""
    import s2cnn_b200 as S
    from s2cnn_b200.soft.so3_fft import SO3_fft_real, SO3_ifft_real, so3_rfft, so3_rifft
    from s2cnn_b200.soft.s2_fft import S2_fft_real, S2_ifft_real
    gen = torch.Generator().manual_seed(11)
    with backends.active(backend) as (_, dev):
        # SO3_fft_real / SO3_ifft_real adjointness:  <A x, y> = <x, A^T y>
        x = torch.randn(2, 8, 8, 8, generator=gen).to(dev).requires_grad_(True)
        y = SO3_fft_real.apply(x, 3)
        gy = torch.randn(y.shape, generator=gen).to(dev)
        y.backward(gy)
        xo = x.detach().cpu().requires_grad_(True)
        yo = O._So3FftReal.apply(xo, 3)
        yo.backward(gy.cpu())
        assert_close(y, yo.detach(), "SO3_fft_real fwd")
        assert_close(x.grad, xo.grad, "SO3_fft_real bwd")

        s = so3_rfft(torch.randn(2, 6, 6, 6, generator=gen).to(dev)).requires_grad_(True)
        out = SO3_ifft_real.apply(s, 4)
        go = torch.randn(out.shape, generator=gen).to(dev)
        out.backward(go)
        so = s.detach().cpu().requires_grad_(True)
        oo = O._So3IfftReal.apply(so, 4)
        oo.backward(go.cpu())
        assert_close(out, oo.detach(), "SO3_ifft_real fwd")
        assert_close(s.grad, so.grad, "SO3_ifft_real bwd")

        x2 = torch.randn(3, 10, 10, generator=gen).to(dev).requires_grad_(True)
        y2 = S2_fft_real.apply(x2, 4)
        g2 = torch.randn(y2.shape, generator=gen).to(dev)
        y2.backward(g2)
        x2o = x2.detach().cpu().requires_grad_(True)
        y2o = O._S2FftReal.apply(x2o, 4)
        y2o.backward(g2.cpu())
        assert_close(y2, y2o.detach(), "S2_fft_real fwd")
        assert_close(x2.grad, x2o.grad, "S2_fft_real bwd")

        sp = torch.randn(9, 2, 2, generator=gen).to(dev)
        assert_close(S2_ifft_real.apply(sp, 5), O.s2_ifft(sp.cpu(), b_out=5)[..., 0], "S2_ifft_real")

        # integrate
        xi = torch.randn(2, 3, 6, 6, 6, generator=gen).to(dev).requires_grad_(True)
        yi = S.so3_integrate(xi)
        yi.sum().backward()
        xio = xi.detach().cpu().requires_grad_(True)
        O.so3_integrate(xio).sum().backward()
        assert_close(xi.grad, xio.grad, "integrate bwd")
        assert_close(S.so3_relu_integrate(xi.detach()), O.so3_integrate(torch.relu(xio.detach())), "relu int")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_small_network_matches_oracle(backend):
    """The benchmark's three-stage classifier at a reduced size: S2Conv -> ReLU -> SO3Conv -> ReLU
    -> so3_integrate -> Linear, forward and parameter gradients against the oracle."""
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3, n_gamma=8)
    torch.manual_seed(3)
    c1 = S.S2Convolution(1, 4, 8, 4, g2)
    c2 = S.SO3Convolution(4, 5, 4, 3, g3)
    lin = torch.nn.Linear(5, 3)
    x = torch.randn(3, 1, 16, 16)
    # oracle
    k1 = c1.kernel.detach().clone().requires_grad_(True)
    k2 = c2.kernel.detach().clone().requires_grad_(True)
    h = torch.relu(O.s2_convolution(x, k1, c1.bias.detach(), 8, 4, g2))
    h = torch.relu(O.so3_convolution(h, k2, c2.bias.detach(), 4, 3, g3))
    yo = torch.nn.functional.linear(O.so3_integrate(h), lin.weight.detach(), lin.bias.detach())
    yo.square().sum().backward()
    with backends.active(backend) as (_, dev):
        c1, c2, lin = c1.to(dev), c2.to(dev), lin.to(dev)
        h = torch.relu(c1(x.to(dev)))
        h = torch.relu(c2(h))
        y = lin(S.so3_integrate(h))
        y.square().sum().backward()
        assert_close(y, yo.detach(), "net out")
        assert_close(c1.kernel.grad, k1.grad, "net gk1")
        assert_close(c2.kernel.grad, k2.grad, "net gk2")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fused_relu_variants_match_unfused(backend):
    """conv(relu(x)) via relu_input=True and so3_relu_integrate equal the unfused composition,
    forward and backward."""
    import s2cnn_b200 as S
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)
    torch.manual_seed(5)
    conv = S.SO3Convolution(2, 3, 4, 3, g3)
    x0 = torch.randn(2, 2, 8, 8, 8)
    with backends.active(backend) as (_, dev):
        conv = conv.to(dev)
        xa = x0.clone().to(dev).requires_grad_(True)
        ya = S.so3_relu_integrate(conv(xa, relu_input=True))
        ya.square().sum().backward()
        ga, gka = xa.grad.clone(), conv.kernel.grad.clone()
        conv.zero_grad()
        xb = x0.clone().to(dev).requires_grad_(True)
        yb = S.so3_integrate(torch.relu(conv(torch.relu(xb))))
        yb.square().sum().backward()
        assert_close(ya, yb.detach(), "fused relu fwd")
        assert_close(ga, xb.grad, "fused relu gx")
        assert_close(gka, conv.kernel.grad, "fused relu gk")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fused_network_paths_match_plain_modules(backend):
    """The inference-only extensions of the modules - ReLU applied on load, the two-layer relay
    (S2Convolution tail + ReLU + SO3Convolution head in one kernel) and ReLU + so3_integrate inside
    the last synthesis - give the same values as the plain chain of modules; with autograd enabled
    the same keyword arguments fall back to that chain."""
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=6, n_beta=2)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)
    torch.manual_seed(21)
    with backends.active(backend) as (_, dev):
        c1 = S.S2Convolution(2, 4, 8, 5, g2).to(dev)
        c2 = S.SO3Convolution(4, 3, 5, 3, g3).to(dev)
        with torch.no_grad():
            c1.bias.copy_(torch.randn(c1.bias.shape))
            c2.bias.copy_(torch.randn(c2.bias.shape))
        x = torch.randn(3, 2, 16, 16).to(dev)
        with torch.no_grad():
            plain = S.so3_integrate(torch.relu(c2(torch.relu(c1(x)))))
            on_load = S.so3_relu_integrate(c2(c1(x), relu_input=True))
            tail = c2(c1(x), relu_input=True, relu_integrate=True)
            relay = c2(c1(x, relu_so3_fft=c2.b_out), input_spectrum=True, relu_integrate=True)
        for name, got in (("relu on load", on_load), ("fused tail", tail), ("relay", relay)):
            assert_close(got, plain.cpu(), name)
        # autograd on: same keywords, gradients flow through the unfused ops
        xg = x.clone().requires_grad_(True)
        y = c2(c1(xg, relu_so3_fft=c2.b_out), input_spectrum=True, relu_integrate=True)
        assert_close(y, plain.cpu(), "relay keywords with autograd")
        y.sum().backward()
        assert xg.grad is not None and torch.isfinite(xg.grad).all()
        assert c1.kernel.grad is not None and c2.kernel.grad is not None
