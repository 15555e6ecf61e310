"""CUDA-graph replay of a forward pass (s2cnn_b200.graph.GraphedForward) reproduces the eager
result, on new inputs and from pinned host memory."""
import numpy as np
import pytest
import torch


@pytest.mark.gpu
def test_graphed_forward_matches_eager():
    import s2cnn_b200 as S
    from s2cnn_b200.graph import GraphedForward
    dev = torch.device("cuda:0")
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)
    torch.manual_seed(1)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = S.S2Convolution(1, 4, 8, 4, g2)
            self.c2 = S.SO3Convolution(4, 6, 4, 3, g3)

        def forward(self, x):
            return S.so3_relu_integrate(self.c2(self.c1(x), relu_input=True))

    net = Net().to(dev).eval()
    gen = torch.Generator().manual_seed(2)
    x0 = torch.randn(5, 1, 16, 16, generator=gen)
    graphed = GraphedForward(net, x0.to(dev))
    for _ in range(2):
        x = torch.randn(5, 1, 16, 16, generator=gen)
        with torch.no_grad():
            ref = net(x.to(dev))
        got = graphed(x.pin_memory()).clone()
        torch.cuda.synchronize()
        assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
