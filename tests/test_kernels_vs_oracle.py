"""Every entry point of the C ABI against the CPU oracle and the reference's golden vectors.

Runs twice: on the host-emulation build of the kernel sources (CPU) and, marked ``gpu``, on the
CUDA library.  Shapes are the ones the reference's own tests use (tests/so3_fft.py:57-102,
s2cnn/soft/s2_fft.py:253-268, s2cnn/s2_mm.py:315-320, s2cnn/so3_mm.py:264-269) plus edge cases:
b = 1, b_out > b_in (zero-padded rows), b_out < b_in (truncation), batch sizes that do not fill a
tile, FFT lengths with prime factors 3, 5, 7, 11, 13.
"""
import glob
import os

import numpy as np
import pytest
import torch

import backends
from oracle import s2cnn_oracle as O
from util import GOLDEN, assert_close, golden, grid_tuple

n3 = O.so3_nspec


def _names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("so3_fft_"))
def test_so3_transforms_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    b_out = int(g["b_out"])
    for fg in (False, True):
        t = "_grad" if fg else ""
        assert_close(ops.so3_rfft(g["x_real"].to(dev), fg, b_out), g["rfft" + t], name + " rfft" + t)
        assert_close(ops.so3_fft(g["x_complex"].to(dev), fg, b_out), g["fft" + t], name + " fft" + t)
        assert_close(ops.so3_ifft(g["spectrum"].to(dev), fg, b_out), g["ifft" + t], name + " ifft" + t)
        assert_close(ops.so3_rifft(g["spectrum"].to(dev), fg, b_out), g["rifft" + t], name + " rifft" + t)
        assert_close(ops.so3_rifft(g["spectrum_h"].to(dev), fg, b_out), g["rifft_h" + t], name + " rifft_h" + t)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,nbatch", [(1, 1, 1), (1, 3, 2), (3, 1, 5), (13, 7, 1),
                                               (6, 6, 37), (8, 8, 3), (5, 12, 2),
                                               # groups of four betas (2b = 24, 28, 32); at 2b = 32
                                               # the single-kernel path runs 512-thread blocks
                                               (12, 12, 5), (14, 9, 4), (16, 16, 5), (16, 10, 6),
                                               (10, 16, 3)])
def test_so3_transforms_oracle(backend, b_in, b_out, nbatch):
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(100 * b_in + b_out)
    x = torch.randn(nbatch, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen)
    s = torch.randn(n3(b_in), nbatch, 2, generator=gen)
    assert_close(ops.so3_rfft(x.to(dev), False, b_out), O.so3_rfft(x, False, b_out), "rfft")
    assert_close(ops.so3_rifft(s.to(dev), False, b_out), O.so3_rifft(s, False, b_out), "rifft")
    assert_close(ops.so3_rifft(s.to(dev), True, b_out), O.so3_rifft(s, True, b_out), "rifft grad")
    assert_close(ops.so3_ifft(s.to(dev), False, b_out), O.so3_ifft(s, False, b_out), "ifft")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_so3_leading_dims_and_bias(backend):
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, 8, 8, 8, generator=gen)
    y = ops.so3_rfft(x.to(dev), b_out=3)
    assert tuple(y.shape) == (n3(3), 2, 3, 2)
    assert_close(y, O.so3_rfft(x, b_out=3), "rfft lead dims")
    s = torch.randn(n3(4), 2, 3, 2, generator=gen)
    bias = torch.randn(3, generator=gen)
    out = ops.so3_rifft(s.to(dev), bias=bias.to(dev))
    assert tuple(out.shape) == (2, 3, 8, 8, 8)
    assert_close(out, O.so3_rifft(s) + bias.view(1, 3, 1, 1, 1), "rifft + bias")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_so3_small_workspace_chunks(backend):
    """A workspace that holds only 2 batch elements forces the chunked path."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(6)
    b_in, b_out, nb = 5, 4, 7
    x = torch.randn(nb, 10, 10, 10, generator=gen).to(dev)
    out = x.new_empty((n3(b_out), nb, 2))
    per = ops.lib.s2c_so3_fft_workspace_min(b_in, b_out)
    ws = torch.empty(2 * per + 8, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream if dev.type == "cuda" else None
    ops.lib.call("s2c_so3_rfft", x.data_ptr(), out.data_ptr(), nb, b_in, b_out, 0,
                 ws.data_ptr(), ws.numel(), stream)
    assert_close(out, O.so3_rfft(x.cpu(), b_out=b_out), "chunked rfft")
    s = torch.randn(n3(b_in), nb, 2, generator=gen).to(dev)
    y = s.new_empty((nb, 8, 8, 8))
    ops.lib.call("s2c_so3_rifft", s.data_ptr(), y.data_ptr(), nb, b_in, b_out, 0, None, 0,
                 ws.data_ptr(), ws.numel(), stream)
    assert_close(y, O.so3_rifft(s.cpu(), b_out=b_out), "chunked rifft")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("s2_fft_"))
def test_s2_fft_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    for fg in (False, True):
        assert_close(ops.s2_fft(g["x"].to(dev), fg, int(g["b_out"])),
                     g["fft_grad" if fg else "fft"], name)
    xr = g["x"][..., 0].contiguous()
    ref = O.s2_fft(torch.stack((xr, torch.zeros_like(xr)), -1), b_out=int(g["b_out"]))
    assert_close(ops.s2_fft(xr.to(dev), b_out=int(g["b_out"]), x_is_real=True), ref, name + " real")
    # real input takes the single-kernel analysis; the two-kernel path must give the same values
    ops.lib.s2c_debug_force_general_path(1)
    try:
        assert_close(ops.s2_fft(xr.to(dev), b_out=int(g["b_out"]), x_is_real=True), ref,
                     name + " real, two kernels")
    finally:
        ops.lib.s2c_debug_force_general_path(0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,nbatch", [(30, 10, 3), (32, 32, 2), (7, 3, 5), (1, 1, 2)])
def test_s2_fft_real_single_kernel(backend, b_in, b_out, nbatch):
    """The single-kernel S2 analysis of a real signal (packed row pairs, generic and two-step row
    FFTs), both weightings, at the first-layer size of the benchmark network among others."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in * 3 + b_out)
    x = torch.randn(nbatch, 2 * b_in, 2 * b_in, generator=gen)
    for fg in (False, True):
        ref = O.s2_fft(torch.stack((x, torch.zeros_like(x)), -1), for_grad=fg, b_out=b_out)
        n0 = ops.lib.s2c_launch_count()
        got = ops.s2_fft(x.to(dev), fg, b_out, x_is_real=True)
        assert ops.lib.s2c_launch_count() - n0 == 1
        assert_close(got, ref, "s2_fft real for_grad=%s" % fg)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("s2_ifft_"))
def test_s2_ifft_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    for fg in (False, True):
        ref = g["ifft_grad" if fg else "ifft"]
        assert_close(ops.s2_ifft(g["x"].to(dev), fg, int(g["b_out"])), ref, name)
        assert_close(ops.s2_ifft(g["x"].to(dev), fg, int(g["b_out"]), out_is_real=True),
                     ref[..., 0], name + " real")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("s2_mm_") + _names("so3_mm_"))
def test_mm_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    fn = ops.s2_mm if name.startswith("s2") else ops.so3_mm
    assert_close(fn(g["x"].to(dev), g["y"].to(dev)), g["z"], name)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("nl,nb,fi,fo", [(4, 2, 3, 5), (3, 70, 5, 9), (1, 1, 1, 1), (5, 3, 18, 2),
                                         (2, 65, 17, 66)])
def test_mm_forward_and_gradients(backend, nl, nb, fi, fo):
    """Forward against the oracle; grad-x / grad-y against autograd through the oracle (which
    equals the reference's hand-written backward kernels, s2cnn/so3_mm.py:95-122)."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(nl * 1000 + nb)
    for so3 in (True, False):
        ns = n3(nl) if so3 else nl * nl
        x = torch.randn(ns, nb, fi, 2, generator=gen, requires_grad=True)
        y = torch.randn(ns, fi, fo, 2, generator=gen, requires_grad=True)
        zo = (O.so3_mm if so3 else O.s2_mm)(x, y)
        gz = torch.randn(zo.shape, generator=gen)
        zo.backward(gz)
        xd, yd, gzd = x.detach().to(dev), y.detach().to(dev), gz.to(dev)
        if so3:
            z, gx, gy = ops.so3_mm(xd, yd), ops.so3_mm_gradx(gzd, yd, nb, fi), ops.so3_mm_grady(gzd, xd, fo)
        else:
            z, gx, gy = ops.s2_mm(xd, yd), ops.s2_mm_gradx(gzd, yd, nb, fi), ops.s2_mm_grady(gzd, xd, fo)
        tag = "so3_mm" if so3 else "s2_mm"
        assert_close(z, zo.detach(), tag)
        assert_close(gx, x.grad, tag + " gradx")
        assert_close(gy, y.grad, tag + " grady")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("nl,nb,fi,fo", [(4, 70, 1, 20), (3, 5, 4, 7), (5, 130, 2, 33), (1, 1, 1, 1)])
def test_s2_mm_gradients_few_input_features(backend, nl, nb, fi, fo):
    """f_in <= 4 takes the streaming gradient kernels (matrix-vector shaped products); they must
    agree with autograd through the oracle and with the tiled kernel every other shape uses."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(nl * 100 + fo)
    x = torch.randn(nl * nl, nb, fi, 2, generator=gen, requires_grad=True)
    y = torch.randn(nl * nl, fi, fo, 2, generator=gen, requires_grad=True)
    zo = O.s2_mm(x, y)
    gz = torch.randn(zo.shape, generator=gen)
    zo.backward(gz)
    xd, yd, gzd = x.detach().to(dev), y.detach().to(dev), gz.to(dev)
    n0 = ops.lib.s2c_launch_count()
    gx, gy = ops.s2_mm_gradx(gzd, yd, nb, fi), ops.s2_mm_grady(gzd, xd, fo)
    assert ops.lib.s2c_launch_count() - n0 == 2
    assert_close(gx, x.grad, "s2_mm gradx")
    assert_close(gy, y.grad, "s2_mm grady")
    ops.lib.s2c_debug_force_general_path(1)
    try:
        assert_close(ops.s2_mm_gradx(gzd, yd, nb, fi), gx.cpu(), "gradx: tiled vs streaming kernel")
        assert_close(ops.s2_mm_grady(gzd, xd, fo), gy.cpu(), "grady: tiled vs streaming kernel")
    finally:
        ops.lib.s2c_debug_force_general_path(0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("s2_rft_") + _names("so3_rft_"))
def test_rft_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    grid = grid_tuple(g["grid"])
    b = int(g["b"])
    F = ops.s2_ft_matrix(b, grid) if name.startswith("s2") else ops.so3_ft_matrix(b, grid)
    F = torch.from_numpy(F).to(dev)
    x = g["x"]
    y = ops.rft_forward(x.reshape(-1, x.size(-1)).to(dev), F)
    assert_close(y.view(-1, *x.shape[:-1], 2), g["y"], name)
    # transpose: <rft(x), g> = <x, rft^T(g)>
    gen = torch.Generator().manual_seed(1)
    gy = torch.randn(y.shape, generator=gen)
    gx = ops.rft_backward(gy.to(dev), F).cpu()
    lhs = (y.cpu().double() * gy.double()).sum().item()
    rhs = (x.reshape(-1, x.size(-1)).double() * gx.double()).sum().item()
    assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), 1.0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_ft_matrices_match_oracle(backend):
    ops, _ = backends.get(backend)
    g3 = O.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3, n_gamma=8)
    for b, grid in [(4, g3), (7, O.so3_equatorial_grid(n_alpha=8)), (3, ((0.0, 0.0, 0.0),))]:
        assert np.abs(ops.so3_ft_matrix(b, grid) - O.so3_ft_matrix(b, grid).numpy()).max() < 1e-6
    for b, grid in [(5, O.s2_near_identity_grid()), (9, O.s2_equatorial_grid(n_alpha=12))]:
        assert np.abs(ops.s2_ft_matrix(b, grid) - O.s2_ft_matrix(b, grid).numpy()).max() < 1e-5


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", _names("so3_integrate_"))
def test_integrate_golden(backend, name):
    ops, dev = backends.get(backend)
    g = golden(name)
    assert_close(ops.so3_integrate(g["x"].to(dev)), g["y"], name)
    b = g["x"].size(-1) // 2
    x = g["x"].clone().requires_grad_(True)
    yo = O.so3_integrate(x)
    gy = torch.randn(yo.shape, generator=torch.Generator().manual_seed(3))
    yo.backward(gy)
    assert_close(ops.so3_integrate_backward(gy.to(dev), b), x.grad, name + " backward")
    # fused activation
    assert_close(ops.so3_integrate(g["x"].to(dev), relu=True), O.so3_integrate(torch.relu(g["x"])), "relu")
    x2 = g["x"].clone().requires_grad_(True)
    O.so3_integrate(torch.relu(x2)).backward(gy)
    assert_close(ops.so3_integrate_backward(gy.to(dev), b, x=g["x"].to(dev), relu=True), x2.grad, "relu bwd")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_write_coverage_no_stale_values(backend):
    """Outputs are fully written: pre-filling them with NaN must leave none behind (the reference
    needs an explicit output[:] = 0 for the Nyquist rows, s2cnn/soft/so3_fft.py:437)."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(9)
    stream = torch.cuda.current_stream().cuda_stream if dev.type == "cuda" else None
    for b_in, b_out in [(3, 5), (5, 3), (4, 4)]:
        nb = 3
        s = torch.randn(n3(b_in), nb, 2, generator=gen).to(dev)
        y = torch.full((nb, 2 * b_out, 2 * b_out, 2 * b_out), float("nan"), device=dev)
        ws = torch.empty(ops.lib.s2c_so3_fft_workspace(nb, b_in, b_out), dtype=torch.uint8, device=dev)
        ops.lib.call("s2c_so3_rifft", s.data_ptr(), y.data_ptr(), nb, b_in, b_out, 0, None, 0,
                     ws.data_ptr(), ws.numel(), stream)
        assert not torch.isnan(y).any()
        x = torch.randn(nb, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen).to(dev)
        o = torch.full((n3(b_out), nb, 2), float("nan"), device=dev)
        ops.lib.call("s2c_so3_rfft", x.data_ptr(), o.data_ptr(), nb, b_in, b_out, 0,
                     ws.data_ptr(), ws.numel(), stream)
        assert not torch.isnan(o).any()


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("name", ["so3_fft_7_5", "so3_fft_4_7", "so3_fft_6_6", "so3_fft_10_11"])
def test_general_three_pass_path_forced(backend, name):
    """Bandwidths up to 16 normally take the single-kernel path; the switch routes them through the
    general three-pass kernels (the path every larger bandwidth uses) so both stay covered."""
    ops, dev = backends.get(backend)
    g = golden(name)
    b_out = int(g["b_out"])
    ops.lib.s2c_debug_force_general_path(1)
    try:
        for fg in (False, True):
            t = "_grad" if fg else ""
            assert_close(ops.so3_rfft(g["x_real"].to(dev), fg, b_out), g["rfft" + t], name + " rfft" + t)
            assert_close(ops.so3_fft(g["x_complex"].to(dev), fg, b_out), g["fft" + t], name + " fft" + t)
            assert_close(ops.so3_ifft(g["spectrum"].to(dev), fg, b_out), g["ifft" + t], name + " ifft" + t)
            assert_close(ops.so3_rifft(g["spectrum"].to(dev), fg, b_out), g["rifft" + t], name + " rifft" + t)
    finally:
        ops.lib.s2c_debug_force_general_path(0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,nbatch", [(17, 17, 2), (20, 8, 3), (9, 18, 1)])
def test_large_bandwidth_general_path(backend, b_in, b_out, nbatch):
    """2b > 32: the general path on its own (FFT lengths 34 = 2*17, 40, 36)."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in)
    x = torch.randn(nbatch, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen)
    s = torch.randn(n3(b_in), nbatch, 2, generator=gen)
    assert_close(ops.so3_rfft(x.to(dev), False, b_out), O.so3_rfft(x, False, b_out), "rfft")
    assert_close(ops.so3_rifft(s.to(dev), False, b_out), O.so3_rifft(s, False, b_out), "rifft")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_rfft_with_relu_on_load(backend):
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(12)
    x = torch.randn(5, 12, 12, 12, generator=gen)
    assert_close(ops.so3_rfft(x.to(dev), b_out=4, relu=True), O.so3_rfft(torch.relu(x), b_out=4), "relu rfft")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,lead", [(6, 6, (3, 2)), (5, 3, (7,)), (16, 16, (2, 3)), (17, 5, (2,))])
def test_rfft_with_per_signal_sums(backend, b_in, b_out, lead):
    """The analysis kernel's by-product (the plain sum of every signal, used for the gradient of
    the bias added at s2cnn/soft/s2_conv.py:45) next to the spectrum itself; 2b = 34 takes the
    two-pass fallback."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(77 + b_in)
    x = torch.randn(*lead, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen) + 0.3
    spec, sums = ops.so3_rfft_with_sums(x.to(dev), for_grad=True, b_out=b_out)
    assert_close(spec, O.so3_rfft(x, True, b_out), "spectrum")
    assert tuple(sums.shape) == tuple(lead)
    assert_close(sums, x.double().sum(dim=(-3, -2, -1)).float(), "per-signal sums")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_spec,b_sig,lead", [(4, 6, (5,)), (6, 6, (2, 3)), (3, 5, (1,)), (10, 16, (2,))])
def test_relu_on_load_gradient_in_the_synthesis_kernel(backend, b_spec, b_sig, lead):
    """Backward of so3_rfft(relu(a), b_out = b_spec): the for_grad synthesis of the spectrum's
    gradient with the ReLU mask applied while storing, against the oracle's two steps (the backward
    of SO3_fft_real, s2cnn/soft/so3_fft.py:453-456, then the mask); a sample of ``a`` that is exactly
    0 gets no gradient (torch's convention for relu)."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(31 + b_spec)
    a = torch.randn(*lead, 2 * b_sig, 2 * b_sig, 2 * b_sig, generator=gen)
    a.view(-1)[::7] = 0.0
    g = torch.randn(n3(b_spec), *lead, 2, generator=gen)
    want = O.so3_rifft(g, True, b_sig) * (a > 0)
    got = ops.so3_rifft_relu_grad(g.to(dev), a.to(dev))
    assert_close(got, want, "masked synthesis")
    assert torch.all(got.cpu()[a <= 0] == 0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,lead", [(6, 6, (5, 3)), (4, 7, (2, 2)), (5, 3, (7,)), (10, 10, (1, 2)),
                                             (16, 16, (3,))])   # 512-thread blocks
def test_synthesis_relu_integrate_fused(backend, b_in, b_out, lead):
    """so3_integrate(relu(so3_rifft(x) + bias)) in the synthesis kernel (the signal is never
    written), incl. a batch count that leaves a partial block."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in * 7 + b_out)
    s = torch.randn(n3(b_in), *lead, 2, generator=gen)
    bias = torch.randn(lead[-1], generator=gen)
    shape = (1,) * (len(lead) - 1) + (lead[-1], 1, 1, 1)
    ref = O.so3_integrate(torch.relu(O.so3_rifft(s, b_out=b_out) + bias.view(shape)))
    got = ops.so3_rifft_relu_integrate(s.to(dev), bias=bias.to(dev), b_out=b_out)
    assert_close(got, ref, "rifft + relu + integrate")
    ref0 = O.so3_integrate(torch.relu(O.so3_rifft(s, b_out=b_out)))
    assert_close(ops.so3_rifft_relu_integrate(s.to(dev), b_out=b_out), ref0, "no bias")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b,b_next,nb,fi,fo", [(4, 3, 3, 2, 3), (6, 6, 5, 1, 4), (10, 6, 2, 1, 6),
                                               (5, 2, 1, 3, 2)])
def test_two_layer_relay_kernel(backend, b, b_next, nb, fi, fo):
    """so3_rfft(relu(so3_rifft(s2_mm(xs, ys)) + bias), b_next) in one kernel against the same chain
    through the oracle."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b * 13 + b_next)
    xs = torch.randn(b * b, nb, fi, 2, generator=gen)
    ys = torch.randn(b * b, fi, fo, 2, generator=gen)
    bias = torch.randn(fo, generator=gen)
    z = O.so3_rifft(O.s2_mm(xs, ys)) + bias.view(1, fo, 1, 1, 1)
    ref = O.so3_rfft(torch.relu(z), b_out=b_next)
    got = ops.s2_conv_relu_so3_rfft(xs.to(dev), ys.to(dev), bias.to(dev), b_next)
    assert_close(got, ref, "relay")
    ref0 = O.so3_rfft(torch.relu(O.so3_rifft(O.s2_mm(xs, ys))), b_out=b_next)
    assert_close(ops.s2_conv_relu_so3_rfft(xs.to(dev), ys.to(dev), None, b_next), ref0, "relay, no bias")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_mid,b_next,lead", [(6, 6, 4, (3, 4)), (4, 7, 5, (2, 3)), (10, 10, 5, (5,)),
                                                     (5, 5, 5, (2, 2))])
def test_relay_kernel_between_so3_layers(backend, b_in, b_mid, b_next, lead):
    """so3_rfft(relu(so3_rifft(x, b_mid) + bias), b_next) in one kernel for a plain spectrum."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in * 17 + b_next)
    x = torch.randn(n3(b_in), *lead, 2, generator=gen)
    bias = torch.randn(lead[-1], generator=gen)
    shape = (1,) * (len(lead) - 1) + (lead[-1], 1, 1, 1)
    ref = O.so3_rfft(torch.relu(O.so3_rifft(x, b_out=b_mid) + bias.view(shape)), b_out=b_next)
    assert_close(ops.so3_rifft_relu_rfft(x.to(dev), bias.to(dev), b_mid, b_next), ref, "relay")
    ref0 = O.so3_rfft(torch.relu(O.so3_rifft(x, b_out=b_mid)), b_out=b_next)
    assert_close(ops.so3_rifft_relu_rfft(x.to(dev), None, b_mid, b_next), ref0, "relay, no bias")


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b,nb,fi,fo", [(4, 3, 2, 3), (6, 5, 1, 4), (1, 2, 3, 2), (10, 2, 1, 6)])
def test_s2_product_synthesis_fused(backend, b, nb, fi, fo):
    """so3_rifft(s2_mm(x, y)) + bias in one call, single-kernel path and general path."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b * 10 + fo)
    xs = torch.randn(b * b, nb, fi, 2, generator=gen)
    ys = torch.randn(b * b, fi, fo, 2, generator=gen)
    bias = torch.randn(fo, generator=gen)
    ref = O.so3_rifft(O.s2_mm(xs, ys)) + bias.view(1, fo, 1, 1, 1)
    assert_close(ops.s2_conv_synthesis(xs.to(dev), ys.to(dev), bias.to(dev)), ref, "fused")
    ops.lib.s2c_debug_force_general_path(1)
    try:
        assert_close(ops.s2_conv_synthesis(xs.to(dev), ys.to(dev), bias.to(dev)), ref, "general")
    finally:
        ops.lib.s2c_debug_force_general_path(0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,nbatch", [(8, 8, 37), (6, 4, 67), (4, 6, 3)])
def test_general_path_tiled_wigner_odd_batches(backend, b_in, b_out, nbatch):
    """The register-tiled Wigner kernels of the general path with batch counts that leave partial
    (and odd) tiles."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in * 31 + nbatch)
    x = torch.randn(nbatch, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen)
    s = torch.randn(n3(b_in), nbatch, 2, generator=gen)
    ops.lib.s2c_debug_force_general_path(1)
    try:
        assert_close(ops.so3_rfft(x.to(dev), False, b_out), O.so3_rfft(x, False, b_out), "rfft")
        assert_close(ops.so3_rifft(s.to(dev), False, b_out), O.so3_rifft(s, False, b_out), "rifft")
        assert_close(ops.so3_fft(torch.stack((x, -x), -1).to(dev), False, b_out),
                     O.so3_fft(torch.stack((x, -x), -1), False, b_out), "fft")
    finally:
        ops.lib.s2c_debug_force_general_path(0)


@pytest.mark.parametrize("backend", backends.BACKENDS)
@pytest.mark.parametrize("b_in,b_out,nbatch", [(32, 32, 1), (32, 9, 3), (10, 32, 2), (32, 34, 2)])
def test_bandwidth_32_two_step_fft(backend, b_in, b_out, nbatch):
    """2b = 64: the large-bandwidth path (plane kernels + the lanes-over-beta Wigner kernels, whole
    batch in one chunk and one or two signals per chunk) and the three separate passes with the
    two-step register FFT (8 x 8) must all agree with the oracle."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(b_in + b_out)
    x = torch.randn(nbatch, 2 * b_in, 2 * b_in, 2 * b_in, generator=gen)
    xc = torch.randn(nbatch, 2 * b_in, 2 * b_in, 2 * b_in, 2, generator=gen)
    s = torch.randn(n3(b_in), nbatch, 2, generator=gen)
    bias = torch.randn(3, generator=gen)
    ref_f, ref_i = O.so3_rfft(x, False, b_out), O.so3_rifft(s, False, b_out)
    ref_c, ref_ic = O.so3_fft(xc, True, b_out), O.so3_ifft(s, True, b_out)
    try:
        for level, width in ((0, 0), (0, 2 if nbatch > 2 else 1), (2, 0)):
            ops.lib.s2c_debug_force_general_path(level)
            ops.lib.s2c_debug_plane_chunk(width)
            tag = " level %d chunk %d" % (level, width)
            assert_close(ops.so3_rfft(x.to(dev), False, b_out), ref_f, "rfft" + tag)
            assert_close(ops.so3_rifft(s.to(dev), False, b_out), ref_i, "rifft" + tag)
            assert_close(ops.so3_fft(xc.to(dev), True, b_out), ref_c, "fft" + tag)
            assert_close(ops.so3_ifft(s.to(dev), True, b_out), ref_ic, "ifft" + tag)
    finally:
        ops.lib.s2c_debug_force_general_path(0)
        ops.lib.s2c_debug_plane_chunk(0)


def test_bandwidth_64_large_path_on_the_emulation_build():
    """2b = 128 (two betas of the half range per lane in the Wigner kernels, 16-point second FFT
    step in the plane kernels) through the host-emulation build, one signal: the GPU twin is
    tests/test_gpu_large_bandwidth.py."""
    ops, dev = backends.get("emul")
    gen = torch.Generator().manual_seed(64)
    x = torch.randn(1, 128, 128, 128, generator=gen)
    ref = O.so3_rfft(x, b_out=64)
    got = ops.so3_rfft(x, b_out=64)
    assert_close(got, ref, "b=64 rfft (emulation)")
    assert_close(ops.so3_rifft(got), O.so3_rifft(ref), "b=64 rifft (emulation)")


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_tensors_aligned_to_16_bytes_only(backend):
    """Signals and spectra whose first element sits 16 bytes into an allocation (a view of a larger
    buffer): the kernels' 32-byte accesses need 32-byte alignment and must not be used then."""
    ops, dev = backends.get(backend)
    gen = torch.Generator().manual_seed(5)
    b = 8
    n = 3 * (2 * b) ** 3
    flat = torch.randn(n + 4, generator=gen).to(dev)
    x = flat[4:].view(3, 2 * b, 2 * b, 2 * b)
    assert x.data_ptr() % 32 == 16 or not x.is_cuda
    spec = ops.so3_rfft(x)
    assert_close(spec, O.so3_rfft(x.cpu()), "rfft of a 16-byte aligned view")
    sflat = torch.randn(n3(b) * 4 * 2 + 4, generator=gen).to(dev)
    s = sflat[4:].view(n3(b), 4, 2)
    got = ops.so3_rifft(s)
    assert_close(got, O.so3_rifft(s.cpu()), "rifft of a 16-byte aligned spectrum")
