"""Multi-rank logic on CPU: world_size 2 over gloo (127.0.0.1).  Covers batch sharding, the
single-bucket gradient all-reduce, the max-over-ranks timing reduction, and that a batch-sharded
layer (run through the host-emulation build) reproduces the unsharded result and gradient."""
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
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import numpy as np
        import backends
        import s2cnn_b200 as S
        from s2cnn_b200 import parallel

        assert parallel.max_over_ranks(1.0 + rank) == float(world)

        grid = S.so3_near_identity_grid(max_beta=np.pi / 8, n_alpha=4, n_beta=2, n_gamma=2)
        torch.manual_seed(0)  # same weights on every rank
        conv = S.SO3Convolution(2, 3, 4, 3, grid)
        x = torch.randn(5, 2, 8, 8, 8, generator=torch.Generator().manual_seed(1))
        gy = torch.randn(5, 3, 6, 6, 6, generator=torch.Generator().manual_seed(2))
        with backends.active("emul"):
            lo, hi = parallel.shard_range(x.size(0), rank, world)
            y = conv(x[lo:hi])
            y.backward(gy[lo:hi])
            n = parallel.allreduce_gradients(conv.parameters())
            assert n == conv.kernel.numel() + conv.bias.numel()
            ref = S.SO3Convolution(2, 3, 4, 3, grid)
            ref.load_state_dict(conv.state_dict())
            yr = ref(x)
            yr.backward(gy)
            out = {"y": y.detach(), "yr": yr[lo:hi].detach(), "gk": conv.kernel.grad.clone(),
                   "gkr": ref.kernel.grad, "gb": conv.bias.grad.clone(), "gbr": ref.bias.grad}

            # a batch of ONE over two ranks: rank 1 owns nothing, runs no backward and must still
            # take part in the collective with the same bucket layout (zeros), and receive the sum
            conv.zero_grad(set_to_none=True)
            lo1, hi1 = parallel.shard_range(1, rank, world)
            if hi1 > lo1:
                conv(x[lo1:hi1]).backward(gy[lo1:hi1])
            else:
                assert conv.kernel.grad is None
            n = parallel.allreduce_gradients(conv.parameters())
            assert n == conv.kernel.numel() + conv.bias.numel()
            ref.zero_grad(set_to_none=True)
            ref(x[:1]).backward(gy[:1])
            out.update({"e_gk": conv.kernel.grad.clone(), "e_gkr": ref.kernel.grad.clone(),
                        "e_gb": conv.bias.grad.clone(), "e_gbr": ref.bias.grad.clone()})

            # the overlapped reducer (one bucket per layer, launched from autograd hooks) on a
            # two-layer stack; second step with rank 1 skipping its backward pass entirely
            torch.manual_seed(5)
            net = torch.nn.Sequential(S.SO3Convolution(2, 3, 4, 3, grid), torch.nn.ReLU(),
                                      S.SO3Convolution(3, 2, 3, 2, grid))
            gy2 = torch.randn(5, 2, 4, 4, 4, generator=torch.Generator().manual_seed(3))
            red = parallel.GradientReducer(net)
            assert len(red.buckets) == 2
            red.zero_grad()
            net(x[lo:hi]).backward(gy2[lo:hi])
            assert red.finish() == sum(p.numel() for p in net.parameters())
            got = [p.grad.clone() for p in net.parameters()]
            red.zero_grad()
            if rank == 0:
                net(x[:2]).backward(gy2[:2])
            red.finish()
            got2 = [p.grad.clone() for p in net.parameters()]
            red.remove()
            for p in net.parameters():
                p.grad = None
            net(x).backward(gy2)
            want = [p.grad.clone() for p in net.parameters()]
            for p in net.parameters():
                p.grad = None
            net(x[:2]).backward(gy2[:2])
            want2 = [p.grad.clone() for p in net.parameters()]
            out.update({"red": got, "red_ref": want, "red2": got2, "red2_ref": want2})
            torch.save(out, os.path.join(tmp, "out%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def test_shard_range_partitions():
    from s2cnn_b200.parallel import shard_range
    for n in (0, 1, 7, 256):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_two_ranks_match_single_process(tmp_path):
    sys.path.insert(0, HERE)
    import emul
    emul.build()  # build once before forking workers
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    from util import assert_close
    for rank in range(2):
        out = torch.load(os.path.join(str(tmp_path), "out%d.pt" % rank))
        assert_close(out["y"], out["yr"], "sharded forward")
        assert_close(out["gk"], out["gkr"], "all-reduced kernel grad")
        assert_close(out["gb"], out["gbr"], "all-reduced bias grad")
        assert_close(out["e_gk"], out["e_gkr"], "kernel grad, rank with an empty shard")
        assert_close(out["e_gb"], out["e_gbr"], "bias grad, rank with an empty shard")
        for a, b in zip(out["red"], out["red_ref"]):
            assert_close(a, b, "overlapped reducer, rank %d" % rank)
        for a, b in zip(out["red2"], out["red2_ref"]):
            assert_close(a, b, "overlapped reducer with an idle rank, rank %d" % rank)


def _timeout_worker(rank, world, port, tmp):
    """Rank 1 never reaches its all-reduce; rank 0 must get a TimeoutError out of finish() instead
    of waiting for ever.  Both leave without touching the (now unusable) process group again."""
    sys.path.insert(0, HERE)
    import backends
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=__import__("datetime").timedelta(seconds=60))
    import s2cnn_b200 as S
    from s2cnn_b200 import parallel
    with backends.active("emul"):
        torch.manual_seed(1)
        grid = S.so3_near_identity_grid(max_beta=0.4, n_alpha=4, n_beta=1, n_gamma=2)
        conv = S.SO3Convolution(2, 2, 3, 2, grid)
        red = parallel.GradientReducer(conv)
        red.zero_grad()
        result = "no finish"
        if rank == 0:
            conv(torch.randn(2, 2, 6, 6, 6)).sum().backward()   # the hook launches the all-reduce
            try:
                red.finish(timeout_s=2.0)
                result = "returned"
            except TimeoutError:
                result = "timeout"
        else:
            import time
            time.sleep(6.0)       # well past rank 0's limit; never joins the collective
        with open(os.path.join(tmp, "timeout%d.txt" % rank), "w") as f:
            f.write(result)
    os._exit(0)


def test_finish_times_out_when_a_rank_never_joins(tmp_path):
    sys.path.insert(0, HERE)
    import emul
    emul.build()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()       # exactly the processes started here
    assert not alive, "a rank hung instead of timing out"
    assert open(os.path.join(str(tmp_path), "timeout0.txt")).read() == "timeout"
    assert open(os.path.join(str(tmp_path), "timeout1.txt")).read() == "no finish"
