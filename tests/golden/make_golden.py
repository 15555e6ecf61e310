"""Generate the golden fixtures in this directory by running the UNMODIFIED reference
(jonkhler/s2cnn, CPU code path) on seeded inputs.

Run from the repository root, on a machine that has a checkout of the reference:

    S2CNN_REFERENCE=/path/to/s2cnn python tests/golden/make_golden.py

The reference is imported through ``oracle/ref_import.py`` (numpy/torch API shims plus the
float64 stand-in for the absent third-party ``lie_learn``; see that file).  Each fixture is
an ``.npz`` holding the inputs and the reference's outputs, so the tests need neither the
reference nor a particular RNG.  Shapes are the ones the reference's own tests use
(tests/so3_fft.py:57-102, s2cnn/soft/s2_fft.py:253-268, s2cnn/s2_mm.py:315-320,
s2cnn/so3_mm.py:264-269).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_import  # noqa: E402

SO3_SHAPES = [(7, 5), (7, 7), (5, 4), (7, 4), (4, 7), (4, 6), (2, 9), (6, 6), (9, 2),
              (10, 11), (11, 10)]


def n3(b):
    return b * (4 * b * b - 1) // 3


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


def rotation_cases():
    """so3_rotation (s2cnn/soft/so3_rotation.py:11-48) with its gradient; own RNG so that
    ``python tests/golden/make_golden.py rotation`` regenerates only these."""
    from s2cnn import so3_rotation
    from s2cnn.soft.so3_rotation import _setup_so3_rotation
    g = torch.Generator().manual_seed(20240608)
    with ref_import.in_scratch():
        for b, nb, abc in ((4, (2, 3), (0.5, 1.0, 0.0)), (7, (2,), (2.1, 0.3, -1.2))):
            x = torch.randn(*nb, 2 * b, 2 * b, 2 * b, generator=g).requires_grad_(True)
            y = so3_rotation(x, *abc)
            gy = torch.randn(*y.shape, generator=g)
            y.backward(gy)
            Us = _setup_so3_rotation(b, *abc, device_type="cpu", device_index=None)
            U = torch.cat([u.reshape(-1, 2) for u in Us], 0)
            save("so3_rotation_%d" % b, b=b, abc=np.array(abc), x=x, y=y, gy=gy, gx=x.grad, U=U)


def main():
    ref = ref_import.load()
    if sys.argv[1:] == ["rotation"]:
        rotation_cases()
        return
    from s2cnn.soft.so3_fft import so3_fft, so3_rfft, so3_ifft, so3_rifft
    from s2cnn.soft.s2_fft import s2_fft, s2_ifft
    import s2cnn

    g = torch.Generator().manual_seed(20240607)

    def randn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    with ref_import.in_scratch():
        # ---- SO(3) transforms, all four, both weightings ---------------------------------
        for b_in, b_out in SO3_SHAPES:
            nb = 2 if max(b_in, b_out) <= 7 else 1
            n = 2 * b_in
            xr = randn(nb, n, n, n)
            xc = randn(nb, n, n, n, 2)
            sp = randn(n3(b_in), nb, 2)
            # a Hermitian-structured spectrum (what real signals produce) for so3_rifft
            sp_h = so3_rfft(randn(nb, n, n, n))
            fx = {}
            for fg in (False, True):
                tag = "_grad" if fg else ""
                fx["rfft" + tag] = so3_rfft(xr, for_grad=fg, b_out=b_out)
                fx["fft" + tag] = so3_fft(xc, for_grad=fg, b_out=b_out)
                fx["ifft" + tag] = so3_ifft(sp, for_grad=fg, b_out=b_out)
                fx["rifft" + tag] = so3_rifft(sp, for_grad=fg, b_out=b_out)
                fx["rifft_h" + tag] = so3_rifft(sp_h, for_grad=fg, b_out=b_out)
            save("so3_fft_%d_%d" % (b_in, b_out), b_in=b_in, b_out=b_out, x_real=xr,
                 x_complex=xc, spectrum=sp, spectrum_h=sp_h, **fx)

        # ---- S2 transforms ---------------------------------------------------------------
        for b_in, b_out in [(6, 5), (6, 6), (5, 2), (12, 12)]:
            x = randn(1, 2, 2 * b_in, 2 * b_in, 2)
            fx = {("fft_grad" if fg else "fft"): s2_fft(x, for_grad=fg, b_out=b_out)
                  for fg in (False, True)}
            save("s2_fft_%d_%d" % (b_in, b_out), b_in=b_in, b_out=b_out, x=x, **fx)
        for b_in, b_out in [(12, 13), (5, 5), (3, 8)]:
            x = randn(b_in * b_in, 3, 2)
            fx = {("ifft_grad" if fg else "ifft"): s2_ifft(x, for_grad=fg, b_out=b_out)
                  for fg in (False, True)}
            save("s2_ifft_%d_%d" % (b_in, b_out), b_in=b_in, b_out=b_out, x=x, **fx)

        # ---- spectral products -----------------------------------------------------------
        for nl, nb, fi, fo in [(4, 2, 3, 5), (6, 3, 2, 4), (1, 1, 1, 1)]:
            x = randn(nl * nl, nb, fi, 2)
            y = randn(nl * nl, fi, fo, 2)
            save("s2_mm_%d_%d_%d_%d" % (nl, nb, fi, fo), x=x, y=y, z=s2cnn.s2_mm(x, y))
            x = randn(n3(nl), nb, fi, 2)
            y = randn(n3(nl), fi, fo, 2)
            save("so3_mm_%d_%d_%d_%d" % (nl, nb, fi, fo), x=x, y=y, z=s2cnn.so3_mm(x, y))

        # ---- kernel-grid -> spectrum -----------------------------------------------------
        s2g = s2cnn.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
        so3g = s2cnn.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8,
                                            n_beta=3, n_gamma=8)
        so3e = s2cnn.so3_equatorial_grid(max_beta=0, max_gamma=0, n_alpha=16, n_beta=1,
                                         n_gamma=1)
        s2e = s2cnn.s2_equatorial_grid(max_beta=0, n_alpha=16, n_beta=1)
        k = randn(2, 3, len(s2g))
        save("s2_rft_near_5", b=5, grid=np.array(s2g), x=k, y=s2cnn.s2_rft(k, 5, s2g))
        k = randn(2, 3, len(s2e))
        save("s2_rft_eq_7", b=7, grid=np.array(s2e), x=k, y=s2cnn.s2_rft(k, 7, s2e))
        k = randn(2, 3, len(so3g))
        save("so3_rft_near_4", b=4, grid=np.array(so3g), x=k, y=s2cnn.so3_rft(k, 4, so3g))
        k = randn(3, 2, len(so3e))
        save("so3_rft_eq_5", b=5, grid=np.array(so3e), x=k, y=s2cnn.so3_rft(k, 5, so3e))
        save("grids",
             s2_near=np.array(s2cnn.s2_near_identity_grid()),
             s2_near_c0=np.array(s2g),
             s2_eq=np.array(s2cnn.s2_equatorial_grid(max_beta=0.2, n_alpha=6, n_beta=3)),
             s2_soft=np.array(s2cnn.s2_soft_grid(3)),
             so3_near=np.array(s2cnn.so3_near_identity_grid()),
             so3_near_c1=np.array(so3g),
             so3_eq=np.array(s2cnn.so3_equatorial_grid(max_beta=0.1, max_gamma=0.3, n_alpha=5,
                                                        n_beta=2, n_gamma=3)),
             so3_soft=np.array(s2cnn.so3_soft_grid(2)))

        # ---- integration -----------------------------------------------------------------
        x = randn(3, 2, 8, 8, 8)
        save("so3_integrate_4", x=x, y=s2cnn.so3_integrate(x))
        x = randn(2, 10, 10, 10)
        save("so3_integrate_5", x=x, y=s2cnn.so3_integrate(x))

        # ---- whole layers with gradients (reference modules, reference autograd rules) ---
        torch.manual_seed(7)
        conv = s2cnn.S2Convolution(2, 3, 6, 4, s2g)
        with torch.no_grad():
            conv.bias.copy_(randn(1, 3, 1, 1, 1))
        x = randn(2, 2, 12, 12).requires_grad_(True)
        y = conv(x)
        gy = randn(*y.shape)
        y.backward(gy)
        save("s2_conv_6_4", b_in=6, b_out=4, grid=np.array(s2g), x=x, kernel=conv.kernel,
             bias=conv.bias, y=y, gy=gy, gx=x.grad, gkernel=conv.kernel.grad,
             gbias=conv.bias.grad)

        conv = s2cnn.SO3Convolution(2, 3, 5, 3, so3g)
        with torch.no_grad():
            conv.bias.copy_(randn(1, 3, 1, 1, 1))
        x = randn(2, 2, 10, 10, 10).requires_grad_(True)
        y = conv(x)
        gy = randn(*y.shape)
        y.backward(gy)
        save("so3_conv_5_3", b_in=5, b_out=3, grid=np.array(so3g), x=x, kernel=conv.kernel,
             bias=conv.bias, y=y, gy=gy, gx=x.grad, gkernel=conv.kernel.grad,
             gbias=conv.bias.grad)

        # SO3Shortcut's one-point grid ((0,0,0),) (s2cnn/soft/so3_conv.py:66-74)
        sc = s2cnn.soft.so3_conv.SO3Shortcut(2, 4, 4, 3)
        x = randn(1, 2, 8, 8, 8)
        save("so3_shortcut_4_3", x=x, kernel=sc.conv.kernel, bias=sc.conv.bias, y=sc(x))

        # ---- tables as the reference builds them (float32, [beta, lmn]) ------------------
        from s2cnn.soft.so3_fft import _setup_so3_fft
        from s2cnn.soft.s2_fft import _setup_s2_fft
        save("tables",
             so3_5_4_w=_setup_so3_fft(5, 4, True), so3_5_4_u=_setup_so3_fft(5, 4, False),
             so3_3_6_w=_setup_so3_fft(3, 6, True),
             s2_6_5_w=_setup_s2_fft(6, 5, True), s2_6_5_u=_setup_s2_fft(6, 5, False))
    rotation_cases()
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
