"""Pointer plumbing between torch tensors and the C ABI (include/s2cnn_b200.h).

``Ops(lib)`` exposes one method per entry point: it checks dtype/shape, allocates the output and
the scratch space with torch (device memory management is all torch is used for here), and passes
raw pointers plus the current CUDA stream.  The public, reference-named API in the sibling modules
is built on ``cuda_ops()``, which is bound to the CUDA build and refuses CPU tensors.
"""
import contextlib
import logging
import os

import torch

from . import _lib


_CHECK_TC = bool(os.environ.get("S2CNN_B200_CHECK_TC"))


def so3_nspec(b):
    return b * (4 * b * b - 1) // 3


def bandwidth_from_so3_nspec(nspec):
    b = round((3.0 / 4.0 * nspec) ** (1.0 / 3.0))  # as s2cnn/soft/so3_fft.py:121-122
    assert nspec == so3_nspec(b), "not an SO(3) spectrum length: %d" % nspec
    return b


def _prod(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class Ops:
    def __init__(self, lib):
        self.lib = lib
        self._tables_seen = 0

    def _log_new_tables(self, what):
        """The reference logs "Compute Wigner ..." on the "trainer" logger whenever a table is
        built (s2cnn/soft/so3_fft.py:223, s2_fft.py:127); same here, from the library's counter."""
        n = self.lib.s2c_tables_computed()
        if n != self._tables_seen:
            logging.getLogger("trainer").info("Compute Wigner tables (%s): %d computed by this process",
                                              what, n)
            self._tables_seen = n

    # -- helpers -------------------------------------------------------------------------------
    def _prep(self, *tensors):
        for t in tensors:
            if t is None:
                continue
            if t.dtype != torch.float32:
                raise TypeError("s2cnn_b200 kernels are float32 only, got %s" % t.dtype)
            if t.is_cuda != self.lib.is_cuda:
                raise _lib.S2cError(
                    "s2cnn_b200: tensor on %s but the loaded library is the %s build - the "
                    "product path runs on CUDA only" % (t.device, "CUDA" if self.lib.is_cuda else "emulation"))

    def _ctx(self, t):
        return torch.cuda.device_of(t) if t.is_cuda else contextlib.nullcontext()

    def _stream(self, t):
        return torch.cuda.current_stream(t.device).cuda_stream if t.is_cuda else None

    @staticmethod
    def _ws(nbytes, like):
        return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=like.device)

    # -- SO(3) transforms ----------------------------------------------------------------------
    def so3_rfft(self, x, for_grad=False, b_out=None, relu=False):
        """[..., 2b, 2b, 2b] real -> [nspec(b_out), ..., 2]; with ``relu`` the transform of
        max(x, 0) (activation applied while reading; small bandwidths, forward weighting only)."""
        self._prep(x)
        b_in = x.size(-1) // 2
        assert x.size(-1) == 2 * b_in and x.size(-2) == 2 * b_in and x.size(-3) == 2 * b_in
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[:-3])
        nbatch = _prod(lead)
        x = x.contiguous()
        out = x.new_empty((so3_nspec(b_out), nbatch, 2))
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_so3_fft_workspace(nbatch, b_in, b_out), x)
            if relu:
                assert not for_grad
                self.lib.call("s2c_so3_rfft_relu", x.data_ptr(), out.data_ptr(), nbatch, b_in,
                              b_out, ws.data_ptr(), ws.numel(), self._stream(x))
            else:
                self.lib.call("s2c_so3_rfft", x.data_ptr(), out.data_ptr(), nbatch, b_in, b_out,
                              int(bool(for_grad)), ws.data_ptr(), ws.numel(), self._stream(x))
        self._log_new_tables("so3_rfft b %d -> %d" % (b_in, b_out))
        return out.view(-1, *lead, 2)

    def so3_rfft_with_sums(self, x, for_grad=False, b_out=None):
        """``so3_rfft(x)`` and, as a by-product of the same kernel, the plain sum of every signal
        over its samples ([...] like the leading dimensions of x).  Sizes outside the single-kernel
        path (2 b_in > 32) take two passes."""
        self._prep(x)
        b_in = x.size(-1) // 2
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[:-3])
        nbatch = _prod(lead)
        x = x.contiguous()
        if 2 * b_in <= 32:
            out = x.new_empty((so3_nspec(b_out), nbatch, 2))
            sums = x.new_empty((nbatch,))
            with self._ctx(x):
                ok = self.lib.try_call("s2c_so3_rfft_sums", x.data_ptr(), out.data_ptr(),
                                       sums.data_ptr(), nbatch, b_in, b_out, int(bool(for_grad)),
                                       self._stream(x))
            if ok:
                self._log_new_tables("so3_rfft b %d -> %d" % (b_in, b_out))
                return out.view(-1, *lead, 2), sums.view(lead)
        return self.so3_rfft(x, for_grad=for_grad, b_out=b_out), x.sum(dim=(-3, -2, -1))

    def so3_fft(self, x, for_grad=False, b_out=None):
        """[..., 2b, 2b, 2b, 2] complex -> [nspec(b_out), ..., 2]"""
        self._prep(x)
        assert x.size(-1) == 2, x.size()
        b_in = x.size(-2) // 2
        assert x.size(-2) == 2 * b_in and x.size(-3) == 2 * b_in and x.size(-4) == 2 * b_in
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[:-4])
        nbatch = _prod(lead)
        x = x.contiguous()
        out = x.new_empty((so3_nspec(b_out), nbatch, 2))
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_so3_fft_workspace(nbatch, b_in, b_out), x)
            self.lib.call("s2c_so3_fft", x.data_ptr(), out.data_ptr(), nbatch, b_in, b_out,
                          int(bool(for_grad)), ws.data_ptr(), ws.numel(), self._stream(x))
        return out.view(-1, *lead, 2)

    def so3_rifft(self, x, for_grad=False, b_out=None, bias=None):
        """[nspec(b_in), ..., 2] -> [..., 2b_out, 2b_out, 2b_out] real (+ per-feature bias, where
        the feature axis is the last leading axis)."""
        self._prep(x, bias)
        assert x.size(-1) == 2
        b_in = bandwidth_from_so3_nspec(x.size(0))
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[1:-1])
        nbatch = _prod(lead)
        x = x.contiguous()
        n = 2 * b_out
        out = x.new_empty((nbatch, n, n, n))
        nfeat = 0
        bias_ptr = None
        if bias is not None:
            bias = bias.contiguous().view(-1)
            nfeat = bias.numel()
            assert len(lead) >= 1 and lead[-1] == nfeat, (lead, nfeat)
            bias_ptr = bias.data_ptr()
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_so3_fft_workspace(nbatch, b_in, b_out), x)
            self.lib.call("s2c_so3_rifft", x.data_ptr(), out.data_ptr(), nbatch, b_in, b_out,
                          int(bool(for_grad)), bias_ptr, nfeat, ws.data_ptr(), ws.numel(),
                          self._stream(x))
        self._log_new_tables("so3_rifft b %d -> %d" % (b_in, b_out))
        return out.view(*lead, n, n, n)

    def so3_rifft_relu_grad(self, x, act):
        """Gradient of ``so3_rfft(relu(act))`` with respect to ``act`` given the gradient ``x`` of the
        spectrum: ``so3_rifft(x, for_grad=True)`` where ``act > 0``, else 0, in one kernel
        (2 b <= 32).  x [nspec(b_in), ..., 2], act [..., 2b, 2b, 2b] -> like act."""
        self._prep(x, act)
        b_in = bandwidth_from_so3_nspec(x.size(0))
        b_out = act.size(-1) // 2
        lead = tuple(act.shape[:-3])
        nbatch = _prod(lead)
        assert tuple(x.shape[1:-1]) == lead and x.size(-1) == 2
        x = x.contiguous()
        act = act.contiguous()
        out = torch.empty_like(act)
        with self._ctx(x):
            self.lib.call("s2c_so3_rifft_relu_grad", x.data_ptr(), act.data_ptr(), out.data_ptr(),
                          nbatch, b_in, b_out, self._stream(x))
        return out

    def so3_rifft_relu_integrate(self, x, bias=None, b_out=None):
        """so3_integrate(relu(so3_rifft(x) + bias)) in one kernel, the signal never written:
        [nspec(b_in), ..., 2] -> [...].  Only 2 b_out <= 32."""
        self._prep(x, bias)
        assert x.size(-1) == 2
        b_in = bandwidth_from_so3_nspec(x.size(0))
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[1:-1])
        nbatch = _prod(lead)
        x = x.contiguous()
        out = x.new_empty((nbatch,))
        nfeat = 0
        bias_ptr = None
        if bias is not None:
            bias = bias.contiguous().view(-1)
            nfeat = bias.numel()
            assert len(lead) >= 1 and lead[-1] == nfeat, (lead, nfeat)
            bias_ptr = bias.data_ptr()
        with self._ctx(x):
            self.lib.call("s2c_so3_rifft_relu_integrate", x.data_ptr(), out.data_ptr(), nbatch,
                          b_in, b_out, bias_ptr, nfeat, self._stream(x))
        return out.view(*lead)

    def s2_conv_relu_so3_rfft(self, xs, ys, bias, b_next):
        """so3_rfft(relu(so3_rifft(s2_mm(xs, ys)) + bias), b_out=b_next) in one kernel (small b).
        xs [b^2, batch, f_in, 2], ys [b^2, f_in, f_out, 2] -> [nspec(b_next), batch, f_out, 2]"""
        self._prep(xs, ys, bias)
        nspec, nbatch, f_in, two = xs.shape
        b = int(round(nspec ** 0.5))
        assert b * b == nspec and two == 2 and tuple(ys.shape[:2]) == (nspec, f_in)
        f_out = ys.size(2)
        xs, ys = xs.contiguous(), ys.contiguous()
        bias_ptr = None
        if bias is not None:
            bias = bias.contiguous().view(-1)
            assert bias.numel() == f_out
            bias_ptr = bias.data_ptr()
        out = xs.new_empty((so3_nspec(b_next), nbatch, f_out, 2))
        with self._ctx(xs):
            self.lib.call("s2c_s2_conv_relu_so3_rfft", xs.data_ptr(), ys.data_ptr(), out.data_ptr(),
                          nbatch, f_in, f_out, b, b_next, bias_ptr, self._stream(xs))
        return out

    def so3_rifft_relu_rfft(self, x, bias, b_mid, b_next):
        """so3_rfft(relu(so3_rifft(x, b_out=b_mid) + bias), b_out=b_next) in one kernel (2 b_mid <= 32).
        x [nspec(b_in), ..., 2] -> [nspec(b_next), ..., 2]"""
        self._prep(x, bias)
        assert x.size(-1) == 2
        b_in = bandwidth_from_so3_nspec(x.size(0))
        lead = tuple(x.shape[1:-1])
        nbatch = _prod(lead)
        x = x.contiguous()
        nfeat = 0
        bias_ptr = None
        if bias is not None:
            bias = bias.contiguous().view(-1)
            nfeat = bias.numel()
            assert len(lead) >= 1 and lead[-1] == nfeat, (lead, nfeat)
            bias_ptr = bias.data_ptr()
        out = x.new_empty((so3_nspec(b_next),) + lead + (2,))
        with self._ctx(x):
            self.lib.call("s2c_so3_rifft_relu_rfft", x.data_ptr(), out.data_ptr(), nbatch, b_in, b_mid,
                          b_next, bias_ptr, nfeat, self._stream(x))
        return out

    def s2_conv_synthesis(self, xs, ys, bias=None):
        """so3_rifft(s2_mm(xs, ys)) + bias without materialising the SO(3) spectrum (small b).
        xs [b^2, batch, f_in, 2], ys [b^2, f_in, f_out, 2] -> [batch, f_out, 2b, 2b, 2b]"""
        self._prep(xs, ys, bias)
        nspec, nbatch, f_in, two = xs.shape
        assert two == 2 and ys.size(0) == nspec and ys.size(1) == f_in and ys.size(3) == 2
        f_out = ys.size(2)
        b = round(nspec ** 0.5)
        assert nspec == b * b
        xs = xs.contiguous()
        ys = ys.contiguous()
        n = 2 * b
        out = xs.new_empty((nbatch, f_out, n, n, n))
        bias_ptr = None
        if bias is not None:
            bias = bias.contiguous().view(-1)
            assert bias.numel() == f_out
            bias_ptr = bias.data_ptr()
        with self._ctx(xs):
            ws = self._ws(self.lib.s2c_s2_conv_synthesis_workspace(nbatch, f_out, b), xs)
            self.lib.call("s2c_s2_conv_synthesis", xs.data_ptr(), ys.data_ptr(), out.data_ptr(),
                          nbatch, f_in, f_out, b, bias_ptr, ws.data_ptr(), ws.numel(),
                          self._stream(xs))
        return out

    def so3_ifft(self, x, for_grad=False, b_out=None):
        """[nspec(b_in), ..., 2] -> [..., 2b_out, 2b_out, 2b_out, 2] complex"""
        self._prep(x)
        assert x.size(-1) == 2
        b_in = bandwidth_from_so3_nspec(x.size(0))
        b_out = b_in if b_out is None else b_out
        lead = tuple(x.shape[1:-1])
        nbatch = _prod(lead)
        x = x.contiguous()
        n = 2 * b_out
        out = x.new_empty((nbatch, n, n, n, 2))
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_so3_fft_workspace(nbatch, b_in, b_out), x)
            self.lib.call("s2c_so3_ifft", x.data_ptr(), out.data_ptr(), nbatch, b_in, b_out,
                          int(bool(for_grad)), ws.data_ptr(), ws.numel(), self._stream(x))
        return out.view(*lead, n, n, n, 2)

    # -- S2 transforms -------------------------------------------------------------------------
    def s2_fft(self, x, for_grad=False, b_out=None, x_is_real=False):
        """[..., 2b, 2b(, 2)] -> [b_out^2, ..., 2]"""
        self._prep(x)
        if x_is_real:
            b_in = x.size(-1) // 2
            assert x.size(-1) == 2 * b_in and x.size(-2) == 2 * b_in
            lead = tuple(x.shape[:-2])
        else:
            assert x.size(-1) == 2
            b_in = x.size(-2) // 2
            assert x.size(-2) == 2 * b_in and x.size(-3) == 2 * b_in
            lead = tuple(x.shape[:-3])
        b_out = b_in if b_out is None else b_out
        assert b_out <= b_in  # s2cnn/soft/s2_fft.py:24
        nbatch = _prod(lead)
        x = x.contiguous()
        out = x.new_empty((b_out * b_out, nbatch, 2))
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_s2_fft_workspace(nbatch, b_in, b_out), x)
            self.lib.call("s2c_s2_fft", x.data_ptr(), int(x_is_real), out.data_ptr(), nbatch, b_in,
                          b_out, int(bool(for_grad)), ws.data_ptr(), ws.numel(), self._stream(x))
        return out.view(-1, *lead, 2)

    def s2_ifft(self, x, for_grad=False, b_out=None, out_is_real=False):
        """[b_in^2, ..., 2] -> [..., 2b_out, 2b_out(, 2)]"""
        self._prep(x)
        assert x.size(-1) == 2
        nspec = x.size(0)
        b_in = round(nspec ** 0.5)
        assert nspec == b_in ** 2
        b_out = b_in if b_out is None else b_out
        assert b_out >= b_in  # s2cnn/soft/s2_fft.py:71
        lead = tuple(x.shape[1:-1])
        nbatch = _prod(lead)
        x = x.contiguous()
        n = 2 * b_out
        shape = (nbatch, n, n) if out_is_real else (nbatch, n, n, 2)
        out = x.new_empty(shape)
        with self._ctx(x):
            ws = self._ws(self.lib.s2c_s2_fft_workspace(nbatch, b_in, b_out), x)
            self.lib.call("s2c_s2_ifft", x.data_ptr(), out.data_ptr(), int(out_is_real), nbatch,
                          b_in, b_out, int(bool(for_grad)), ws.data_ptr(), ws.numel(),
                          self._stream(x))
        return out.view(*lead, *shape[1:])

    # -- spectral products ---------------------------------------------------------------------
    def _mm(self, fn, a, b, out_shape, nl, nbatch, f_in, f_out):
        self._prep(a, b)
        a = a.contiguous()
        b = b.contiguous()
        out = a.new_empty(out_shape)
        with self._ctx(a):
            self.lib.call(fn, a.data_ptr(), b.data_ptr(), out.data_ptr(), nl, nbatch, f_in, f_out,
                          self._stream(a))
            if _CHECK_TC and self.lib.is_cuda:
                self.check_tensor_core_status()
        return out

    def check_tensor_core_status(self):
        """Waits for the device and raises if a tensor-core product has given up on one of its
        bounded barrier waits since the library was loaded (its output is then undefined).  Called
        after every spectral product when the environment variable S2CNN_B200_CHECK_TC is set; a
        training loop can call it once per step instead."""
        rc = self.lib.s2c_so3_mm_tc_status()
        if rc != 0:
            raise _lib.S2cError("s2cnn_b200: a tensor-core spectral product reported a barrier "
                                "time-out (status %d); its results are invalid" % rc)

    @staticmethod
    def _mm_dims(x_shape, y_shape, so3):
        nspec, nbatch, f_in, two = x_shape
        assert two == 2 and y_shape[3] == 2
        f_out = y_shape[2]
        assert y_shape[1] == f_in and y_shape[0] == nspec
        if so3:
            nl = bandwidth_from_so3_nspec(nspec)
        else:
            nl = round(nspec ** 0.5)
            assert nspec == nl * nl
        return nl, nbatch, f_in, f_out

    def so3_mm(self, x, y):
        nl, nb, fi, fo = self._mm_dims(x.shape, y.shape, True)
        return self._mm("s2c_so3_mm", x, y, (so3_nspec(nl), nb, fo, 2), nl, nb, fi, fo)

    def so3_mm_gradx(self, gz, y, nb, fi):
        nl = bandwidth_from_so3_nspec(y.size(0))
        fo = y.size(2)
        return self._mm("s2c_so3_mm_gradx", gz, y, (so3_nspec(nl), nb, fi, 2), nl, nb, fi, fo)

    def so3_mm_grady(self, gz, x, fo):
        nl = bandwidth_from_so3_nspec(x.size(0))
        nb, fi = x.size(1), x.size(2)
        return self._mm("s2c_so3_mm_grady", gz, x, (so3_nspec(nl), fi, fo, 2), nl, nb, fi, fo)

    def s2_mm(self, x, y):
        nl, nb, fi, fo = self._mm_dims(x.shape, y.shape, False)
        return self._mm("s2c_s2_mm", x, y, (so3_nspec(nl), nb, fo, 2), nl, nb, fi, fo)

    def s2_mm_gradx(self, gz, y, nb, fi):
        nl = round(y.size(0) ** 0.5)
        fo = y.size(2)
        return self._mm("s2c_s2_mm_gradx", gz, y, (nl * nl, nb, fi, 2), nl, nb, fi, fo)

    def s2_mm_grady(self, gz, x, fo):
        nl = round(x.size(0) ** 0.5)
        nb, fi = x.size(1), x.size(2)
        return self._mm("s2c_s2_mm_grady", gz, x, (nl * nl, fi, fo, 2), nl, nb, fi, fo)

    # -- kernel-grid -> spectrum ---------------------------------------------------------------
    def rft_forward(self, x2d, F):
        """x2d [nf, n_grid], F [n_grid, nspec, 2] -> [nspec, nf, 2]"""
        self._prep(x2d, F)
        nf, ng = x2d.shape
        assert F.size(0) == ng and F.size(2) == 2
        ns = F.size(1)
        x2d = x2d.contiguous()
        F = F.contiguous()
        out = x2d.new_empty((ns, nf, 2))
        with self._ctx(x2d):
            self.lib.call("s2c_rft_forward", x2d.data_ptr(), F.data_ptr(), out.data_ptr(), nf, ng,
                          ns, self._stream(x2d))
        return out

    def rft_forward_t(self, x2d, Ft):
        """The same product on the tensor cores: x2d [nf, n_grid], Ft [nspec, 2, n_grid] (the
        transposed Fourier matrix) -> [nspec, nf, 2].  CUDA build, even n_grid."""
        self._prep(x2d, Ft)
        nf, ng = x2d.shape
        assert Ft.size(2) == ng and Ft.size(1) == 2
        ns = Ft.size(0)
        x2d = x2d.contiguous()
        Ft = Ft.contiguous()
        out = x2d.new_empty((ns, nf, 2))
        with self._ctx(x2d):
            self.lib.call("s2c_rft_forward_t", x2d.data_ptr(), Ft.data_ptr(), out.data_ptr(), nf, ng,
                          ns, self._stream(x2d))
        return out

    def rft_backward(self, g, F):
        """g [nspec, nf, 2], F [n_grid, nspec, 2] -> [nf, n_grid]"""
        self._prep(g, F)
        ns, nf, _ = g.shape
        ng = F.size(0)
        assert F.size(1) == ns
        g = g.contiguous()
        F = F.contiguous()
        out = g.new_empty((nf, ng))
        with self._ctx(g):
            self.lib.call("s2c_rft_backward", g.data_ptr(), F.data_ptr(), out.data_ptr(), nf, ng,
                          ns, self._stream(g))
        return out

    # -- integration ---------------------------------------------------------------------------
    def so3_integrate(self, x, relu=False):
        self._prep(x)
        assert x.size(-1) == x.size(-2) and x.size(-2) == x.size(-3)
        b = x.size(-1) // 2
        lead = tuple(x.shape[:-3])
        n = _prod(lead)
        x = x.contiguous()
        out = x.new_empty((n,))
        with self._ctx(x):
            self.lib.call("s2c_so3_integrate", x.data_ptr(), out.data_ptr(), n, b, int(relu),
                          self._stream(x))
        return out.view(*lead)

    def so3_integrate_backward(self, g, b, x=None, relu=False):
        self._prep(g, x)
        lead = tuple(g.shape)
        n = _prod(lead)
        g = g.contiguous()
        if x is not None:
            x = x.contiguous()
        m = 2 * b
        out = g.new_empty((n, m, m, m))
        with self._ctx(g):
            self.lib.call("s2c_so3_integrate_backward", g.data_ptr(),
                          x.data_ptr() if x is not None else None, out.data_ptr(), n, b,
                          int(relu), self._stream(g))
        return out.view(*lead, m, m, m)

    # -- host generators -----------------------------------------------------------------------
    def so3_rotation_matrices(self, b, alpha, beta, gamma):
        """Host: concatenated Wigner-D matrices [b(4b^2-1)/3, 2] of one rotation."""
        import numpy as np
        U = np.empty((so3_nspec(b), 2), dtype=np.float32)
        self.lib.call("s2c_so3_rotation_matrices", b, float(alpha), float(beta), float(gamma),
                      U.ctypes.data)
        return U

    def so3_rotate_spectrum(self, U, x, b, adjoint=False):
        """x [nspec3, ..., 2] -> rotated spectrum of the same shape (adjoint: transposed map)."""
        self._prep(U, x)
        if x.shape[0] != so3_nspec(b) or x.shape[-1] != 2 or tuple(U.shape) != (so3_nspec(b), 2):
            raise ValueError("so3_rotate_spectrum: bad shapes")
        x = x.contiguous()
        nbatch = _prod(tuple(x.shape[1:-1]))
        out = torch.empty_like(x)
        with self._ctx(x):
            self.lib.call("s2c_so3_rotate_spectrum", U.data_ptr(), x.data_ptr(), out.data_ptr(), b,
                          nbatch, int(adjoint), self._stream(x))
        return out

    # -- data preparation ----------------------------------------------------------------------
    def project_on_sphere(self, verts, faces, grid):
        """verts [nv, 3] float32, faces [nf, 3] int32, grid [nr, 3] float32 -> [3, nr] float32
        (distance to the first hit, normal . ray, |normal x ray|; see include/s2cnn_b200.h)."""
        self._prep(verts, grid)
        if faces.dtype != torch.int32 or faces.is_cuda != self.lib.is_cuda:
            raise TypeError("faces must be an int32 tensor on the library's device")
        assert verts.dim() == 2 and verts.size(1) == 3 and faces.dim() == 2 and faces.size(1) == 3
        assert grid.dim() == 2 and grid.size(1) == 3
        assert int(faces.min()) >= 0 and int(faces.max()) < verts.size(0), "face index out of range"
        verts, faces, grid = verts.contiguous(), faces.contiguous(), grid.contiguous()
        out = verts.new_empty((3, grid.size(0)))
        with self._ctx(verts):
            self.lib.call("s2c_project_on_sphere", verts.data_ptr(), verts.size(0), faces.data_ptr(),
                          faces.size(0), grid.data_ptr(), grid.size(0), out.data_ptr(),
                          self._stream(verts))
        return out

    def so3_ft_matrix(self, b, grid):
        import numpy as np
        g = np.ascontiguousarray(np.asarray(grid, dtype=np.float64).reshape(len(grid), 3))
        F = np.empty((len(grid), so3_nspec(b), 2), dtype=np.float32)
        self.lib.call("s2c_so3_ft_matrix", b, g.ctypes.data, len(grid), F.ctypes.data)
        return F

    def s2_ft_matrix(self, b, grid):
        import numpy as np
        g = np.ascontiguousarray(np.asarray(grid, dtype=np.float64).reshape(len(grid), 2))
        F = np.empty((len(grid), b * b, 2), dtype=np.float32)
        self.lib.call("s2c_s2_ft_matrix", b, g.ctypes.data, len(grid), F.ctypes.data)
        return F


_cuda_ops = None


def cuda_ops():
    global _cuda_ops
    if _cuda_ops is None:
        _cuda_ops = Ops(_lib.cuda_lib())
    return _cuda_ops
