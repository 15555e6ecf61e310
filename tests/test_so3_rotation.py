"""so3_rotation (s2cnn/soft/so3_rotation.py:11-73): the oracle against the reference's outputs,
the CUDA / emulated kernels against both, and the property the reference's
examples/equivariance_plot/main.py:74-78 demonstrates - an SO(3) convolution commutes with a
general rotation of its input."""
import importlib

import pytest
import torch

import backends
from oracle import s2cnn_oracle as O
from util import assert_close, golden

CASES = ["so3_rotation_4", "so3_rotation_7"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference(name):
    g = golden(name)
    b, abc = int(g["b"]), [float(v) for v in g["abc"]]
    U = O.so3_rotation_matrices(b, *abc)
    assert_close(torch.view_as_real(torch.from_numpy(U)), g["U"], name + " U")
    x = g["x"].clone().requires_grad_(True)
    y = O.so3_rotation(x, *abc)
    assert_close(y, g["y"], name + " y")
    y.backward(g["gy"])
    assert_close(x.grad, g["gx"], name + " gx")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", CASES)
def test_kernels_match_reference(backend, name):
    import s2cnn_b200
    mod = importlib.import_module("s2cnn_b200.soft.so3_rotation")
    g = golden(name)
    b, abc = int(g["b"]), [float(v) for v in g["abc"]]
    with backends.active(backend) as (ops, dev):
        mod._setup_so3_rotation.cache_clear()
        assert_close(torch.from_numpy(ops.so3_rotation_matrices(b, *abc)), g["U"], name + " U")
        x = g["x"].clone().to(dev).requires_grad_(True)
        y = s2cnn_b200.so3_rotation(x, *abc)
        assert y.shape == x.shape
        assert_close(y, g["y"], name + " y")
        y.backward(g["gy"].to(dev))
        assert_close(x.grad, g["gx"], name + " gx")
        mod._setup_so3_rotation.cache_clear()


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_rotation_composes_and_inverts(backend):
    """R(-c,-b,-a) undoes R(a,b,c) on band-limited signals (U is unitary)."""
    import s2cnn_b200
    mod = importlib.import_module("s2cnn_b200.soft.so3_rotation")
    b = 5
    gen = torch.Generator().manual_seed(3)
    with backends.active(backend) as (ops, dev):
        mod._setup_so3_rotation.cache_clear()
        spec = torch.randn(O.so3_nspec(b), 3, 2, generator=gen)
        x = O.so3_rifft(spec).to(dev)                    # band-limited real signal
        y = s2cnn_b200.so3_rotation(x, 0.7, 1.1, -0.4)
        back = s2cnn_b200.so3_rotation(y, 0.4, -1.1, -0.7)
        # the real synthesis keeps the Hermitian part, which x already is
        assert_close(back, O.so3_rifft(O.so3_rfft(x.cpu())), "inverse rotation")
        mod._setup_so3_rotation.cache_clear()


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_so3_convolution_is_equivariant_to_general_rotations(backend):
    import s2cnn_b200
    mod = importlib.import_module("s2cnn_b200.soft.so3_rotation")
    b = 5
    abc = (0.5, 1.0, 0.3)
    gen = torch.Generator().manual_seed(11)
    grid = s2cnn_b200.so3_near_identity_grid(max_beta=0.2, n_alpha=6, n_beta=1, n_gamma=2)
    with backends.active(backend) as (ops, dev):
        mod._setup_so3_rotation.cache_clear()
        conv = s2cnn_b200.SO3Convolution(2, 3, b, b, grid)
        with torch.no_grad():
            conv.kernel.copy_(torch.randn(conv.kernel.shape, generator=gen))
            conv.bias.zero_()
        conv = conv.to(dev)
        spec = torch.randn(O.so3_nspec(b), 1, 2, 2, generator=gen)
        x = O.so3_rifft(spec).to(dev)                    # [1, 2, 2b, 2b, 2b], band-limited
        with torch.no_grad():
            y1 = conv(s2cnn_b200.so3_rotation(x, *abc))
            y2 = s2cnn_b200.so3_rotation(conv(x), *abc)
        err = (y1 - y2).std().item() / y1.std().item()
        assert err < 1e-4, err
        mod._setup_so3_rotation.cache_clear()
