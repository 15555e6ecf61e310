"""The batch-sharded training step on real GPUs: two ranks over NCCL (127.0.0.1), each running the
CUDA library on its half of the batch and reducing the parameter gradients - once with one blocking
all-reduce after backward, once with per-layer all-reduces launched from autograd hooks;
rank 0 checks outputs and gradients against the unsharded step.  Skipped when fewer than two GPUs
are visible (the CPU twin of this test is test_parallel_gloo.py)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import numpy as np
        import s2cnn_b200 as S
        from s2cnn_b200 import parallel

        assert parallel.max_over_ranks(1.0 + rank, device=dev) == float(world)
        g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
        g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)

        def make():
            torch.manual_seed(0)  # same weights on every rank
            return torch.nn.ModuleList([S.S2Convolution(2, 6, 10, 5, g2),
                                        S.SO3Convolution(6, 4, 5, 3, g3)]).to(dev)

        def forward(net, x):
            return S.so3_integrate(torch.relu(net[1](torch.relu(net[0](x)))))

        x = torch.randn(6, 2, 20, 20, generator=torch.Generator().manual_seed(1)).to(dev)
        gy = torch.randn(6, 4, generator=torch.Generator().manual_seed(2)).to(dev)
        net = make()
        lo, hi = parallel.shard_range(x.size(0), rank, world)
        y = forward(net, x[lo:hi])
        y.backward(gy[lo:hi])
        n = parallel.allreduce_gradients(net.parameters())
        assert n == sum(p.numel() for p in net.parameters())
        torch.cuda.synchronize()
        blocking = [p.grad.clone() for p in net.parameters()]
        # the same step with the per-layer all-reduces launched from autograd hooks during backward
        red = parallel.GradientReducer(net)
        assert len(red.buckets) == 2
        red.zero_grad()
        forward(net, x[lo:hi]).backward(gy[lo:hi])
        assert red.finish() == n
        torch.cuda.synchronize()
        overlapped = [p.grad.clone() for p in net.parameters()]
        red.remove()
        if rank == 0:
            ref = make()
            yr = forward(ref, x)
            yr.backward(gy)
            out = {"y": y.detach().cpu(), "yr": yr[lo:hi].detach().cpu()}
            for i, q in enumerate(ref.parameters()):
                out["g%d" % i] = blocking[i].cpu()
                out["o%d" % i] = overlapped[i].cpu()
                out["r%d" % i] = q.grad.cpu()
            torch.save(out, os.path.join(tmp, "out.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_rank_training_step_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    out = torch.load(os.path.join(str(tmp_path), "out.pt"))
    from util import assert_close
    assert_close(out["y"], out["yr"], "sharded forward")
    i = 0
    while "g%d" % i in out:
        assert_close(out["g%d" % i], out["r%d" % i], "reduced gradient %d" % i)
        assert_close(out["o%d" % i], out["r%d" % i], "gradient %d reduced from hooks" % i)
        i += 1
    assert i == 4
