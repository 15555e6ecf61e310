"""The tcgen05 / TMEM implementation of so3_mm (3xTF32) against the oracle, on shapes that
exercise: the benchmark layer (nl 6, batch 256, 20 -> 40), several K blocks per p (2 f_in > 48),
row tiles that straddle m, partial row and column tiles, one degree only, odd feature counts
(8-byte accesses) and the last layer of the reference's deep configuration (100 -> 255).  GPU only - the
kernel has no host emulation; the FP32 kernel it replaces is checked on both builds elsewhere."""
import pytest
import torch

from oracle import s2cnn_oracle as O
from util import assert_close

n3 = O.so3_nspec


@pytest.mark.gpu
@pytest.mark.parametrize("nl,nb,fi,fo", [(6, 256, 20, 40), (3, 130, 26, 6), (4, 100, 4, 64),
                                         (1, 1, 2, 2), (5, 3, 18, 2), (2, 300, 50, 10),
                                         (4, 33, 7, 9), (3, 5, 1, 1), (5, 32, 100, 255)])
def test_so3_mm_tensor_core_matches_oracle(nl, nb, fi, fo):
    from s2cnn_b200 import _lib
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    gen = torch.Generator().manual_seed(nl * 7 + fi)
    x = torch.randn(n3(nl), nb, fi, 2, generator=gen)
    y = torch.randn(n3(nl), fi, fo, 2, generator=gen)
    z = ops.so3_mm(x.cuda(), y.cuda())
    torch.cuda.synchronize()
    assert _lib.cuda_lib().s2c_so3_mm_tc_status() == 0
    assert_close(z, O.so3_mm(x, y), "so3_mm tcgen05")
    # and it agrees with the FP32 FMA kernel it replaces
    _lib.cuda_lib().s2c_debug_force_general_path(1)
    try:
        z_simt = ops.so3_mm(x.cuda(), y.cuda())
    finally:
        _lib.cuda_lib().s2c_debug_force_general_path(0)
    assert_close(z, z_simt, "tcgen05 vs FP32 kernel")


def _grad_reference(x, y, gz, nl):
    """Gradients of z = so3_mm(x, y) by complex arithmetic in float64 (s2cnn/so3_mm.py:40-61):
    gx[l,m,p,i,k] = sum_{n,j} gz[l,m,n,i,j] y[l,n,p,k,j],  gy[l,n,p,k,j] = sum_{m,i} conj(gz) x."""
    xc = torch.view_as_complex(x.double().contiguous())
    yc = torch.view_as_complex(y.double().contiguous())
    gc = torch.view_as_complex(gz.double().contiguous())
    gx, gy = torch.zeros_like(xc), torch.zeros_like(yc)
    for l in range(nl):
        L, o = 2 * l + 1, O.so3_offset(l)
        xl = xc[o:o + L * L].reshape(L, L, *xc.shape[1:])      # [m, p, i, k]
        yl = yc[o:o + L * L].reshape(L, L, *yc.shape[1:])      # [n, p, k, j]
        gl = gc[o:o + L * L].reshape(L, L, *gc.shape[1:])      # [m, n, i, j]
        gx[o:o + L * L] = torch.einsum("mnij,npkj->mpik", gl, yl).reshape(L * L, *xc.shape[1:])
        gy[o:o + L * L] = torch.einsum("mnij,mpik->npkj", gl.conj(), xl).reshape(L * L, *yc.shape[1:])
    return torch.view_as_real(gx).float(), torch.view_as_real(gy).float()


@pytest.mark.gpu
@pytest.mark.parametrize("nl,nb,fi,fo", [(6, 256, 20, 40), (3, 130, 26, 6), (4, 100, 4, 64),
                                         (1, 2, 2, 2), (5, 4, 18, 2), (2, 300, 50, 10),
                                         (3, 64, 7, 10), (4, 33, 7, 9), (3, 5, 1, 1),
                                         (5, 32, 100, 255)])
def test_so3_mm_gradients_on_tensor_cores(nl, nb, fi, fo):
    """Both gradient products through the same tcgen05 kernel (row / column addressing and sign
    pattern per product) against float64 complex arithmetic and against the FP32 kernel; odd feature
    counts or batches take the variant with 8-byte accesses."""
    from s2cnn_b200 import _lib
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    lib = _lib.cuda_lib()
    gen = torch.Generator().manual_seed(nl * 11 + fo)
    x = torch.randn(n3(nl), nb, fi, 2, generator=gen)
    y = torch.randn(n3(nl), fi, fo, 2, generator=gen)
    gz = torch.randn(n3(nl), nb, fo, 2, generator=gen)
    ref_gx, ref_gy = _grad_reference(x, y, gz, nl)
    n0 = lib.s2c_launch_count()
    gx = ops.so3_mm_gradx(gz.cuda(), y.cuda(), nb, fi)
    gy = ops.so3_mm_grady(gz.cuda(), x.cuda(), fo)
    torch.cuda.synchronize()
    assert lib.s2c_launch_count() - n0 == 2
    assert lib.s2c_so3_mm_tc_status() == 0
    assert_close(gx, ref_gx, "grad x")
    assert_close(gy, ref_gy, "grad y")
    lib.s2c_debug_force_general_path(1)
    try:
        gx_simt = ops.so3_mm_gradx(gz.cuda(), y.cuda(), nb, fi)
        gy_simt = ops.so3_mm_grady(gz.cuda(), x.cuda(), fo)
    finally:
        lib.s2c_debug_force_general_path(0)
    assert_close(gx, gx_simt, "grad x: tcgen05 vs FP32 kernel")
    assert_close(gy, gy_simt, "grad y: tcgen05 vs FP32 kernel")


@pytest.mark.gpu
@pytest.mark.parametrize("nf,ng,b,so3", [(20, 24, 10, False), (800, 192, 6, True), (600, 24, 16, False),
                                         (130, 192, 10, True), (7, 2, 3, True), (64, 128, 5, True)])
def test_kernel_transform_on_tensor_cores_matches_fp32_kernel_and_oracle(nf, ng, b, so3):
    """s2_rft / so3_rft as a plain real product on the tcgen05 pipeline (forward with the transposed
    Fourier matrix, backward with the row operand read as strided pairs) against the FP32 kernels and
    a float64 einsum; sizes: the bench layers, the deep model's first layer, ragged tiles, a two-point
    grid, an equatorial ring of 128 points."""
    from s2cnn_b200 import _lib
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    ns = n3(b) if so3 else b * b
    gen = torch.Generator().manual_seed(nf + ng)
    x = torch.randn(nf, ng, generator=gen)
    F = torch.randn(ng, ns, 2, generator=gen)
    g = torch.randn(ns, nf, 2, generator=gen)
    want = torch.einsum("fa,asc->sfc", x.double(), F.double()).float()
    want_b = torch.einsum("sfc,asc->fa", g.double(), F.double()).float()
    xd, Fd, gd = x.cuda(), F.cuda(), g.cuda()
    Ft = Fd.permute(1, 2, 0).contiguous()
    got = ops.rft_forward_t(xd, Ft)
    got_b = ops.rft_backward(gd, Fd)
    torch.cuda.synchronize()
    assert _lib.cuda_lib().s2c_so3_mm_tc_status() == 0
    assert_close(got, want, "rft forward on tensor cores")
    assert_close(got_b, want_b, "rft backward on tensor cores")
    assert_close(ops.rft_forward(xd, Fd), want, "rft forward FP32 kernel")
    _lib.cuda_lib().s2c_debug_force_general_path(1)
    try:
        assert_close(ops.rft_backward(gd, Fd), want_b, "rft backward FP32 kernel")
    finally:
        _lib.cuda_lib().s2c_debug_force_general_path(0)
