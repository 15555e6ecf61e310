"""``s2cnn_b200.fuse``: a model written the way the reference's examples write theirs (module calls,
``F.relu``, ``so3_integrate`` in a hand-written ``forward`` - examples/mnist/run.py:55-98) is
rewritten into the fused kernels and still computes the same function: against the unfused model,
and against the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import backends
from util import assert_close


def _model(S, b_in=8, b1=4, b2=3, f1=5, f2=6, nout=4, three=False):
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = S.S2Convolution(nfeature_in=2, nfeature_out=f1, b_in=b_in, b_out=b1, grid=g2)
            self.conv2 = S.SO3Convolution(nfeature_in=f1, nfeature_out=f2, b_in=b1, b_out=b2, grid=g3)
            if three:
                self.conv3 = S.SO3Convolution(nfeature_in=f2, nfeature_out=f2, b_in=b2, b_out=b2, grid=g3)
            self.out_layer = nn.Linear(f2, nout)

        def forward(self, x):
            x = self.conv1(x)
            x = F.relu(x)
            x = self.conv2(x)
            x = F.relu(x)
            if three:
                x = self.conv3(x)
                x = torch.relu(x)
            x = S.so3_integrate(x)
            x = self.out_layer(x)
            return x

    return Net(), g2, g3


@pytest.mark.parametrize("three", [False, True])
@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fused_model_matches_plain_model_and_oracle(backend, three):
    import s2cnn_b200 as S
    from oracle import s2cnn_oracle as O
    with backends.active(backend) as (ops, dev):
        torch.manual_seed(11)
        net, g2, g3 = _model(S, three=three)
        with torch.no_grad():
            for m in net.modules():
                if hasattr(m, "bias") and isinstance(m, (S.S2Convolution, S.SO3Convolution)):
                    m.bias.normal_()
        x = torch.randn(3, 2, 16, 16)
        with torch.no_grad():
            h = torch.relu(O.s2_convolution(x, net.conv1.kernel, net.conv1.bias, 8, 4, g2))
            h = torch.relu(O.so3_convolution(h, net.conv2.kernel, net.conv2.bias, 4, 3, g3))
            if three:
                h = torch.relu(O.so3_convolution(h, net.conv3.kernel, net.conv3.bias, 3, 3, g3))
            want = net.out_layer(O.so3_integrate(h))
        net = net.to(dev).eval()
        fused = S.fuse(net)
        code = fused.code
        assert "relu_so3_fft" in code and "input_spectrum = True" in code
        assert "relu_integrate = True" in code
        assert "relu(" not in code and "so3_integrate" not in code
        xd = x.to(dev)
        with torch.no_grad():
            plain = net(xd)
            n0 = ops.lib.s2c_launch_count()
            got = fused(xd)
            n_fused = ops.lib.s2c_launch_count() - n0
            n0 = ops.lib.s2c_launch_count()
            net(xd)
            n_plain = ops.lib.s2c_launch_count() - n0
        assert n_fused < n_plain
        assert_close(got, plain, "fused vs plain model")
        assert_close(got, want, "fused model vs oracle")
        # the traced model shares the parameters: training through it reaches the same tensors
        fused.train()
        y = fused(xd)
        y.square().sum().backward()
        g_fused = net.conv1.kernel.grad.clone()
        net.zero_grad()
        net(xd).square().sum().backward()
        assert_close(g_fused, net.conv1.kernel.grad, "gradient through the fused model")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fuse_leaves_shared_activations_alone(backend):
    """A pre-activation tensor with a second consumer must stay in memory: no rewrite there."""
    import s2cnn_b200 as S
    with backends.active(backend) as (ops, dev):
        g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)

        class Res(nn.Module):
            def __init__(self):
                super().__init__()
                self.a = S.SO3Convolution(2, 2, 3, 3, g3)
                self.b = S.SO3Convolution(2, 2, 3, 3, g3)

            def forward(self, x):
                y = self.a(x)
                z = self.b(F.relu(y))
                return S.so3_integrate(F.relu(z + y))

        torch.manual_seed(3)
        net = Res().to(dev).eval()
        fused = S.fuse(net)
        assert "relu_so3_fft" not in fused.code and "input_spectrum" not in fused.code
        assert "so3_relu_integrate" in fused.code      # relu -> integrate of a plain tensor
        x = torch.randn(2, 2, 6, 6, 6).to(dev)
        with torch.no_grad():
            assert_close(fused(x), net(x), "residual model")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fuse_folds_eval_mode_batchnorm(backend):
    """conv -> BatchNorm3d -> ReLU -> conv -> BatchNorm3d -> ReLU -> so3_integrate, the layout of the
    reference's 3-D shape model (examples/shrec17/model.py:17-35): in eval mode the normalisations
    disappear into the layers and the chains fuse; in training mode nothing is folded."""
    import s2cnn_b200 as S
    with backends.active(backend) as (ops, dev):
        g2 = S.s2_equatorial_grid(max_beta=0, n_alpha=8, n_beta=1)
        g3 = S.so3_equatorial_grid(max_beta=0, max_gamma=0, n_alpha=8, n_beta=1, n_gamma=1)
        torch.manual_seed(21)

        class Net(nn.Module):
            def __init__(self):
                super().__init__()
                self.sequential = nn.Sequential(
                    S.S2Convolution(3, 5, 8, 4, g2), nn.BatchNorm3d(5, affine=True), nn.ReLU(),
                    S.SO3Convolution(5, 4, 4, 3, g3), nn.BatchNorm3d(4, affine=True), nn.ReLU())
                self.out_layer = nn.Linear(4, 3)

            def forward(self, x):
                x = self.sequential(x)
                x = S.so3_integrate(x)
                return F.log_softmax(self.out_layer(x), dim=1)

        net = Net()
        with torch.no_grad():
            for m in net.modules():
                if isinstance(m, nn.BatchNorm3d):
                    m.running_mean.normal_()
                    m.running_var.uniform_(0.5, 2.0)
                    m.weight.normal_()
                    m.bias.normal_()
                if isinstance(m, (S.S2Convolution, S.SO3Convolution)):
                    m.bias.normal_()
        net = net.to(dev)
        x = torch.randn(3, 3, 16, 16).to(dev)
        net.train()
        assert "channel_scale" not in S.fuse(net).code          # batch statistics: not foldable
        net.eval()
        fused = S.fuse(net)
        code = fused.code
        assert "channel_scale" in code and "relu_so3_fft" in code and "relu_integrate = True" in code
        assert "sequential_1(" not in code and "sequential_4(" not in code     # no BatchNorm call left
        with torch.no_grad():
            assert_close(fused(x), net(x), "model with folded BatchNorm3d")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_fused_training_recompute_rule_gives_the_same_gradients(backend):
    """With ``fused_training`` the fused kernels run in a training step too (the signal between the
    layers is not kept; backward recomputes it through the unfused chain): same loss, same input,
    kernel and bias gradients as the plain model."""
    import s2cnn_b200 as S
    with backends.active(backend) as (ops, dev):
        torch.manual_seed(31)
        net, _, _ = _model(S, three=True)
        net = net.to(dev)
        x = torch.randn(3, 2, 16, 16).to(dev).requires_grad_(True)
        net(x).square().sum().backward()
        want = [x.grad.clone()] + [p.grad.clone() for p in net.parameters()]
        x.grad = None
        net.zero_grad()
        fused = S.fuse(net)
        for m in net.modules():
            if isinstance(m, (S.S2Convolution, S.SO3Convolution)):
                m.fused_training = True
        n0 = ops.lib.s2c_launch_count()
        loss = fused(x).square().sum()
        n_fwd = ops.lib.s2c_launch_count() - n0
        loss.backward()
        got = [x.grad.clone()] + [p.grad.clone() for p in net.parameters()]
        for a, b in zip(got, want):
            assert_close(a, b, "gradient through the recompute rule")
        for m in net.modules():
            if isinstance(m, (S.S2Convolution, S.SO3Convolution)):
                m.fused_training = False
        n0 = ops.lib.s2c_launch_count()
        fused(x)
        assert n_fwd < ops.lib.s2c_launch_count() - n0     # the training forward really was the fused one
