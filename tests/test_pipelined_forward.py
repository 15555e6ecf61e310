"""PipelinedForward / InterleavedForward: graph replays overlapped with uploads and with each other
must return, for every batch of a sequence of different batches, exactly what the module returns
for it."""
import numpy as np
import pytest
import torch


def _net(dev):
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    torch.manual_seed(5)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = S.S2Convolution(1, 4, 10, 5, g2)
            self.c2 = S.SO3Convolution(4, 6, 5, 3, g3)

        def forward(self, x):
            return S.so3_relu_integrate(self.c2(self.c1(x), relu_input=True))

    return Net().to(dev).eval()


@pytest.mark.gpu
def test_pipelined_forward_matches_module_outputs():
    from s2cnn_b200.graph import PipelinedForward
    dev = torch.device("cuda:0")
    net = _net(dev)
    gen = torch.Generator().manual_seed(9)
    batches = [torch.randn(8, 1, 20, 20, generator=gen).pin_memory() for _ in range(7)]
    results = [torch.empty(8, 6).pin_memory() for _ in batches]
    pipe = PipelinedForward(net, batches[0].to(dev))
    for x, y in zip(batches, results):
        pipe.submit(x, y)
    pipe.wait()
    with torch.no_grad():
        for x, y in zip(batches, results):
            ref = net(x.to(dev)).cpu()
            assert torch.equal(y, ref) or (y - ref).abs().max() <= 1e-6 * ref.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("lanes", [1, 2, 3])
def test_interleaved_forward_matches_module_outputs(lanes):
    from s2cnn_b200.graph import InterleavedForward
    dev = torch.device("cuda:0")
    net = _net(dev)
    gen = torch.Generator().manual_seed(19)
    batches = [torch.randn(8, 1, 20, 20, generator=gen).to(dev) for _ in range(7)]
    fwd = InterleavedForward(net, batches[0], lanes=lanes)
    got = []
    fwd.fork()
    for i, x in enumerate(batches):
        lane = fwd.submit(x)
        # the lane's output buffer is overwritten by its next submit: copy it out on the lane's stream
        with torch.cuda.stream(fwd.streams[lane]):
            got.append(fwd.output(lane).clone())
    fwd.join()
    torch.cuda.synchronize()
    with torch.no_grad():
        for x, y in zip(batches, got):
            ref = net(x)
            assert torch.equal(y, ref) or (y - ref).abs().max() <= 1e-6 * ref.abs().max()
