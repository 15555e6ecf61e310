"""The networks of the reference's examples as importable modules, built from this package's
layers.  Attribute names and ``nn.Sequential`` positions are the reference's, so its checkpoints
(``state_dict``) load unchanged:

* ``S2ConvNet_original``  - examples/mnist/run.py:55-98   (conv1, conv2, out_layer)
* ``S2ConvNet_deep``      - examples/mnist/run.py:101-185 (convolutional.{0,2,...,12}, linear.{0,...,7})
* ``Shrec17Model``        - examples/shrec17/model.py:7-48 (sequential.{0,...}, out_layer)

Every model is written with plain module calls; ``s2cnn_b200.fuse(model)`` routes the conv - ReLU
- conv and conv - ReLU - so3_integrate chains through the fused kernels (and folds an eval-mode
BatchNorm3d that follows a convolution into that layer's spectrum and bias).
"""
import numpy as np
import torch.nn as nn
import torch.nn.functional as F

from .s2_grid import s2_equatorial_grid, s2_near_identity_grid
from .so3_grid import so3_equatorial_grid, so3_near_identity_grid
from .soft.s2_conv import S2Convolution
from .soft.so3_conv import SO3Convolution
from .soft.so3_integrate import so3_integrate


class S2ConvNet_original(nn.Module):
    """Spherical-MNIST classifier: S2Conv(1 -> 20, b 30 -> 10), ReLU, SO3Conv(20 -> 40, b 10 -> 6),
    ReLU, so3_integrate, Linear(40 -> 10); default near-identity grids."""

    def __init__(self, f1=20, f2=40, f_output=10, b_in=30, b_l1=10, b_l2=6):
        super().__init__()
        self.conv1 = S2Convolution(nfeature_in=1, nfeature_out=f1, b_in=b_in, b_out=b_l1,
                                   grid=s2_near_identity_grid())
        self.conv2 = SO3Convolution(nfeature_in=f1, nfeature_out=f2, b_in=b_l1, b_out=b_l2,
                                    grid=so3_near_identity_grid())
        self.out_layer = nn.Linear(f2, f_output)

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.relu(self.conv2(x))
        return self.out_layer(so3_integrate(x))


class S2ConvNet_deep(nn.Module):
    """Seven convolutions with bandwidth halving every other layer and a three-layer head with
    BatchNorm1d; kernel grids widen (max_beta pi/16 ... pi/2) as the bandwidth shrinks."""

    def __init__(self, bandwidth=30):
        super().__init__()
        b = bandwidth

        def so3_grid(max_beta):
            return so3_near_identity_grid(n_alpha=6, max_beta=max_beta, n_beta=1, max_gamma=2 * np.pi,
                                          n_gamma=6)

        g1, g2, g3, g4 = so3_grid(np.pi / 16), so3_grid(np.pi / 8), so3_grid(np.pi / 4), so3_grid(np.pi / 2)
        # (f_in, f_out, b_in, b_out, grid) of the six SO(3) layers after the S2 layer 1 -> 8
        plan = [(8, 16, b, b // 2, g1), (16, 16, b // 2, b // 2, g2), (16, 24, b // 2, b // 4, g2),
                (24, 24, b // 4, b // 4, g3), (24, 32, b // 4, b // 8, g3), (32, 64, b // 8, b // 8, g4)]
        layers = [S2Convolution(nfeature_in=1, nfeature_out=8, b_in=b, b_out=b,
                                grid=s2_near_identity_grid(n_alpha=6, max_beta=np.pi / 16, n_beta=1)),
                  nn.ReLU(inplace=False)]
        for fi, fo, bi, bo, grid in plan:
            layers += [SO3Convolution(nfeature_in=fi, nfeature_out=fo, b_in=bi, b_out=bo, grid=grid),
                       nn.ReLU(inplace=False)]
        self.convolutional = nn.Sequential(*layers)
        self.linear = nn.Sequential(
            nn.BatchNorm1d(64), nn.Linear(64, 64), nn.ReLU(inplace=False),
            nn.BatchNorm1d(64), nn.Linear(64, 32), nn.ReLU(inplace=False),
            nn.BatchNorm1d(32), nn.Linear(32, 10))

    def forward(self, x):
        return self.linear(so3_integrate(self.convolutional(x)))


class Shrec17Model(nn.Module):
    """3-D shape classifier on six spherical channels (s2cnn_b200.projection.ProjectOnSphere):
    S2Conv(6 -> 100, b 64 -> 16), [BatchNorm3d, ReLU, SO3Conv(100 -> 100, b 16 -> 10)],
    BatchNorm3d, ReLU, so3_integrate, Linear(100 -> nclasses), log-softmax; equatorial ring kernels
    with 2 b_in points."""

    def __init__(self, nclasses, features=(6, 100, 100), bandwidths=(64, 16, 10)):
        super().__init__()
        self.features = list(features) + [nclasses]
        self.bandwidths = list(bandwidths)
        assert len(self.bandwidths) == len(self.features) - 1
        seq = [S2Convolution(self.features[0], self.features[1], self.bandwidths[0], self.bandwidths[1],
                             s2_equatorial_grid(max_beta=0, n_alpha=2 * self.bandwidths[0], n_beta=1))]
        for l in range(1, len(self.features) - 2):
            f_in, f_out = self.features[l], self.features[l + 1]
            b_in, b_out = self.bandwidths[l], self.bandwidths[l + 1]
            seq += [nn.BatchNorm3d(f_in, affine=True), nn.ReLU(),
                    SO3Convolution(f_in, f_out, b_in, b_out,
                                   so3_equatorial_grid(max_beta=0, max_gamma=0, n_alpha=2 * b_in,
                                                       n_beta=1, n_gamma=1))]
        seq += [nn.BatchNorm3d(self.features[-2], affine=True), nn.ReLU()]
        self.sequential = nn.Sequential(*seq)
        self.out_layer = nn.Linear(self.features[-2], self.features[-1])

    def forward(self, x):
        x = so3_integrate(self.sequential(x))
        return F.log_softmax(self.out_layer(x), dim=1)
