"""The oracle (oracle/s2cnn_oracle.py) against golden vectors produced by the reference
itself (tests/golden/make_golden.py).  CPU only."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import s2cnn_oracle as O
from oracle import wigner_np
from util import GOLDEN, assert_close, golden, grid_tuple


def _names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("name", _names("so3_fft_"))
def test_so3_transforms(name):
    g = golden(name)
    b_out = int(g["b_out"])
    for fg in (False, True):
        t = "_grad" if fg else ""
        assert_close(O.so3_rfft(g["x_real"], fg, b_out), g["rfft" + t], name + " rfft" + t)
        assert_close(O.so3_fft(g["x_complex"], fg, b_out), g["fft" + t], name + " fft" + t)
        assert_close(O.so3_ifft(g["spectrum"], fg, b_out), g["ifft" + t], name + " ifft" + t)
        assert_close(O.so3_rifft(g["spectrum"], fg, b_out), g["rifft" + t], name + " rifft" + t)
        assert_close(O.so3_rifft(g["spectrum_h"], fg, b_out), g["rifft_h" + t], name + " rifft_h" + t)


@pytest.mark.parametrize("name", _names("s2_fft_"))
def test_s2_fft(name):
    g = golden(name)
    for fg in (False, True):
        assert_close(O.s2_fft(g["x"], fg, int(g["b_out"])), g["fft_grad" if fg else "fft"], name)


@pytest.mark.parametrize("name", _names("s2_ifft_"))
def test_s2_ifft(name):
    g = golden(name)
    for fg in (False, True):
        assert_close(O.s2_ifft(g["x"], fg, int(g["b_out"])), g["ifft_grad" if fg else "ifft"], name)


@pytest.mark.parametrize("name", _names("s2_mm_"))
def test_s2_mm(name):
    g = golden(name)
    assert_close(O.s2_mm(g["x"], g["y"]), g["z"], name)


@pytest.mark.parametrize("name", _names("so3_mm_"))
def test_so3_mm(name):
    g = golden(name)
    assert_close(O.so3_mm(g["x"], g["y"]), g["z"], name)


@pytest.mark.parametrize("name", _names("s2_rft_"))
def test_s2_rft(name):
    g = golden(name)
    assert_close(O.s2_rft(g["x"], int(g["b"]), grid_tuple(g["grid"])), g["y"], name)


@pytest.mark.parametrize("name", _names("so3_rft_"))
def test_so3_rft(name):
    g = golden(name)
    assert_close(O.so3_rft(g["x"], int(g["b"]), grid_tuple(g["grid"])), g["y"], name)


@pytest.mark.parametrize("name", _names("so3_integrate_"))
def test_so3_integrate(name):
    g = golden(name)
    assert_close(O.so3_integrate(g["x"]), g["y"], name)


def test_grids_bit_identical():
    g = golden("grids")
    pairs = {
        "s2_near": O.s2_near_identity_grid(),
        "s2_near_c0": O.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3),
        "s2_eq": O.s2_equatorial_grid(max_beta=0.2, n_alpha=6, n_beta=3),
        "s2_soft": O.s2_soft_grid(3),
        "so3_near": O.so3_near_identity_grid(),
        "so3_near_c1": O.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi,
                                                n_alpha=8, n_beta=3, n_gamma=8),
        "so3_eq": O.so3_equatorial_grid(max_beta=0.1, max_gamma=0.3, n_alpha=5, n_beta=2, n_gamma=3),
        "so3_soft": O.so3_soft_grid(2),
    }
    for k, mine in pairs.items():
        ref = g[k].numpy() if hasattr(g[k], "numpy") else g[k]
        assert np.array_equal(np.array(mine), ref), k  # float64, bit for bit


def _conv_case(name, fn):
    g = golden(name)
    x = g["x"].clone().requires_grad_(True)
    k = g["kernel"].clone().requires_grad_(True)
    bias = g["bias"].clone().requires_grad_(True)
    y = fn(x, k, bias, int(g["b_in"]), int(g["b_out"]), grid_tuple(g["grid"]))
    assert_close(y, g["y"], name + " y")
    y.backward(g["gy"])
    assert_close(x.grad, g["gx"], name + " gx")
    assert_close(k.grad, g["gkernel"], name + " gkernel")
    assert_close(bias.grad, g["gbias"], name + " gbias")


def test_s2_convolution_layer():
    _conv_case("s2_conv_6_4", O.s2_convolution)


def test_so3_convolution_layer():
    _conv_case("so3_conv_5_3", O.so3_convolution)


def test_so3_shortcut():
    g = golden("so3_shortcut_4_3")
    y = O.so3_convolution(g["x"], g["kernel"], g["bias"], 4, 3, ((0, 0, 0),))
    assert_close(y, g["y"], "shortcut")


def test_tables_match_reference_layout():
    g = golden("tables")
    assert_close(O.so3_wigner_table(5, 4, True), g["so3_5_4_w"].float(), "so3 w")
    assert_close(O.so3_wigner_table(5, 4, False), g["so3_5_4_u"].float(), "so3 u")
    assert_close(O.so3_wigner_table(3, 6, True), g["so3_3_6_w"].float(), "so3 3->6")
    assert_close(O.s2_wigner_table(6, 5, True), g["s2_6_5_w"].float(), "s2 w")
    assert_close(O.s2_wigner_table(6, 5, False), g["s2_6_5_u"].float(), "s2 u")


def test_wigner_known_answers():
    beta = 0.37
    d1 = wigner_np.wigner_d_matrix(1, beta)
    assert abs(d1[1, 1] - np.cos(beta)) < 1e-14
    assert abs(d1[2, 1] + np.sin(beta) / np.sqrt(2)) < 1e-14
    assert np.allclose(wigner_np.wigner_d_matrix(5, 0.0), np.eye(11), atol=1e-13)
    for b in (2, 5, 16):
        w = wigner_np.quadrature_weights(b)
        assert abs(w.sum() * (2 * b) ** 2 - 1) < 1e-13
    # orthogonality pinned by the reference's round-trip tests (tests/so3_fft.py:34-91)
    b = 6
    w = wigner_np.quadrature_weights(b)
    betas = wigner_np.soft_betas(b)
    for l1 in range(b):
        for l2 in range(b):
            s = sum(w[j] * wigner_np.wigner_d_matrix(l1, betas[j])[l1, l1 + 0]
                    * wigner_np.wigner_d_matrix(l2, betas[j])[l2, l2 + 0] for j in range(2 * b))
            expect = 1.0 / ((2 * b) ** 2 * (2 * l1 + 1)) if l1 == l2 else 0.0
            assert abs(s - expect) < 1e-13


def test_reference_round_trip_property():
    """The reference's idempotence test (tests/so3_fft.py:34-54) on the oracle."""
    torch.manual_seed(0)
    for b_in, b_out in [(7, 7), (5, 4), (4, 6)]:
        x = torch.randn(2 * b_in, 2 * b_in, 2 * b_in)
        x1 = O.so3_rifft(O.so3_rfft(x, b_out=b_out), b_out=b_in)
        x2 = O.so3_rifft(O.so3_rfft(x1, b_out=b_out), b_out=b_in)
        assert (x1 - x2).abs().max().item() < 1e-4 * x2.abs().mean().item()
