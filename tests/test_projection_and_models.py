"""Callers on either side of the spectral path: the ray-cast projection of a mesh onto the sphere
grid (the CUDA replacement of examples/shrec17/dataset.py:render_model) against its numpy
restatement and against cases with a known answer, the on-disk table cache, and the reference's
example networks as importable modules."""
import multiprocessing as mp
import os

import numpy as np
import pytest
import torch

import backends
from util import assert_close


def _icosphere(radius=0.6, subdivisions=2):
    """A triangulated sphere with outward-oriented faces."""
    t = (1.0 + 5 ** 0.5) / 2.0
    v = np.array([[-1, t, 0], [1, t, 0], [-1, -t, 0], [1, -t, 0], [0, -1, t], [0, 1, t], [0, -1, -t],
                  [0, 1, -t], [t, 0, -1], [t, 0, 1], [-t, 0, -1], [-t, 0, 1]], dtype=np.float64)
    f = np.array([[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11], [1, 5, 9], [5, 11, 4],
                  [11, 10, 2], [10, 7, 6], [7, 1, 8], [3, 9, 4], [3, 4, 2], [3, 2, 6], [3, 6, 8],
                  [3, 8, 9], [4, 9, 5], [2, 4, 11], [6, 2, 10], [8, 6, 7], [9, 8, 1]])
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    for _ in range(subdivisions):
        cache, nf = {}, []
        vl = list(v)

        def mid(a, b):
            key = (min(a, b), max(a, b))
            if key not in cache:
                m = vl[a] + vl[b]
                vl.append(m / np.linalg.norm(m))
                cache[key] = len(vl) - 1
            return cache[key]

        for a, b, c in f:
            ab, bc, ca = mid(a, b), mid(b, c), mid(c, a)
            nf += [[a, ab, ca], [b, bc, ab], [c, ca, bc], [ab, bc, ca]]
        v, f = np.array(vl), np.array(nf)
    return v * radius, f


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_projection_matches_numpy_restatement_and_analytic_cases(backend):
    from oracle import projection_np
    from s2cnn_b200 import projection as P
    ops, dev = backends.get(backend)
    b = 6
    sgrid = P.make_sgrid(b, 0.3, 0.7, 1.1)
    assert sgrid.shape == (4 * b * b, 3) and np.allclose(np.linalg.norm(sgrid, axis=1), 1.0)
    rng = np.random.default_rng(5)
    v, f = _icosphere(0.6, 2)
    v = v * (1.0 + 0.3 * rng.standard_normal((len(v), 1)) * 0.2) + np.array([0.05, -0.02, 0.03])
    want = projection_np.render_model(v, f, sgrid)
    got = ops.project_on_sphere(torch.tensor(v, dtype=torch.float32, device=dev),
                                torch.tensor(f, dtype=torch.int32, device=dev),
                                torch.tensor(sgrid, dtype=torch.float32, device=dev)).cpu().double()
    # a ray within rounding distance of an edge may pick either neighbour: allow a handful of such
    # rays, all others agree to float32 accuracy
    bad = (np.abs(got.numpy() - want) > 2e-4).any(axis=0)
    assert bad.sum() <= 2, bad.sum()
    # an exact sphere of radius r around the origin, seen along a face centre: distance 1 - r_face
    v0, f0 = _icosphere(0.5, 0)
    centre = v0[f0[0]].mean(axis=0)
    grid = np.stack((centre / np.linalg.norm(centre), np.array([0.0, 0.0, 1.0])))
    out = ops.project_on_sphere(torch.tensor(v0, dtype=torch.float32, device=dev),
                                torch.tensor(f0, dtype=torch.int32, device=dev),
                                torch.tensor(grid, dtype=torch.float32, device=dev)).cpu().numpy()
    assert abs(out[0, 0] - (1.0 - np.linalg.norm(centre))) < 1e-5     # distance to that face
    assert abs(out[1, 0] - 1.0) < 1e-5 and abs(out[2, 0]) < 1e-3      # normal parallel to the ray
    # a mesh far off to the side is missed by every ray: distance 1, the other channels 0
    miss = ops.project_on_sphere(torch.tensor(v0 * 0.01 + 5.0, dtype=torch.float32, device=dev),
                                 torch.tensor(f0, dtype=torch.int32, device=dev),
                                 torch.tensor(grid, dtype=torch.float32, device=dev)).cpu().numpy()
    assert np.array_equal(miss, np.array([[1.0, 1.0], [0.0, 0.0], [0.0, 0.0]], dtype=np.float32))


@pytest.mark.gpu
def test_project_on_sphere_six_channels_feed_the_shape_model():
    """mesh -> ProjectOnSphere -> Shrec17Model (fused) at the reference's sizes, batch 1: shapes,
    the normalisation constants, fused == plain, and log-probabilities that sum to one."""
    import s2cnn_b200 as S
    from oracle import projection_np
    v, f = _icosphere(0.8, 3)
    proj = S.projection.ProjectOnSphere(64)
    im = proj(v, f)
    assert tuple(im.shape) == (6, 128, 128) and im.dtype == torch.float32
    raw = projection_np.render_model(v, f, proj.sgrid)
    want0 = (raw[0] - 0.75) / 0.26
    ok = np.abs(im[0].reshape(-1).cpu().numpy() - want0) < 1e-3
    assert ok.mean() > 0.999
    torch.manual_seed(0)
    net = S.models.Shrec17Model(nclasses=7).cuda().eval()
    keys = set(net.state_dict())
    assert {"sequential.0.kernel", "sequential.0.bias", "sequential.1.running_mean",
            "sequential.3.kernel", "sequential.4.weight", "out_layer.weight"} <= keys
    x = im.unsqueeze(0)
    with torch.no_grad():
        plain = net(x)
        fused = S.fuse(net)(x)
    assert tuple(plain.shape) == (1, 7)
    assert abs(float(plain.exp().sum()) - 1.0) < 1e-4
    assert_close(fused, plain, "fused shape model")


@pytest.mark.gpu
def test_mnist_models_construct_and_run():
    import s2cnn_b200 as S
    torch.manual_seed(1)
    net = S.models.S2ConvNet_original().cuda().eval()
    assert set(net.state_dict()) == {"conv1.kernel", "conv1.bias", "conv2.kernel", "conv2.bias",
                                     "out_layer.weight", "out_layer.bias"}
    x = torch.randn(4, 1, 60, 60, device="cuda")
    with torch.no_grad():
        assert_close(S.fuse(net)(x), net(x), "S2ConvNet_original fused")
    deep = S.models.S2ConvNet_deep(bandwidth=16).cuda().eval()
    assert "convolutional.12.kernel" in deep.state_dict() and "linear.7.weight" in deep.state_dict()
    xd = torch.randn(3, 1, 32, 32, device="cuda")
    with torch.no_grad():
        yd = deep(xd)
        assert tuple(yd.shape) == (3, 10)
        assert_close(S.fuse(deep)(xd), yd, "S2ConvNet_deep fused")


def _cache_worker(path, build, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from s2cnn_b200 import _lib
    from s2cnn_b200.ops import Ops
    ops = Ops(_lib.Lib(build))
    ops.lib.s2c_set_table_cache_dir(os.fsencode(path))
    x = torch.randn(2, 16, 16, 16, generator=torch.Generator().manual_seed(3))
    y = ops.so3_rfft(x, b_out=6)
    q.put((float(y.abs().sum()), ops.lib.s2c_table_cache_hits(), ops.lib.s2c_table_cache_stores()))


def test_table_disk_cache_shared_by_processes(tmp_path):
    """Two processes start at once on an empty cache directory, both compute (or one reads what the
    other has just finished), both get the same spectrum; a third process finds the file and
    computes nothing; a damaged file is detected by its checksum and replaced."""
    import emul
    build = emul.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cache_worker, args=(str(tmp_path), build, q)) for _ in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join()
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[0][0])
    files = sorted(os.listdir(tmp_path))
    assert files and all(name.endswith(".s2ct") for name in files), files    # no temporaries left
    p3 = ctx.Process(target=_cache_worker, args=(str(tmp_path), build, q))
    p3.start()
    total, hits, stores = q.get(timeout=300)
    p3.join()
    assert hits >= 1 and stores == 0 and abs(total - res[0][0]) <= 1e-6 * abs(total)
    victim = os.path.join(tmp_path, files[0])
    with open(victim, "r+b") as fh:
        fh.seek(os.path.getsize(victim) - 8)
        fh.write(b"\xff" * 8)
    p4 = ctx.Process(target=_cache_worker, args=(str(tmp_path), build, q))
    p4.start()
    total4, hits4, stores4 = q.get(timeout=300)
    p4.join()
    assert stores4 >= 1 and abs(total4 - res[0][0]) <= 1e-6 * abs(total4)
