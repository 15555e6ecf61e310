"""Bandwidth 64 (the standalone-FFT benchmark size, 2b = 128: plane kernels + lanes-over-beta
Wigner kernels in L2-sized batch chunks, checked against the three separate passes with the two-step
8 x 16 register FFT) on the GPU: spectrum parity against the oracle for one batch element, the reference's idempotence
property of the round trip (tests/so3_fft.py:34-44) and linearity at a larger batch."""
import pytest
import torch

from oracle import s2cnn_oracle as O
from util import assert_close


@pytest.mark.gpu
def test_b64_spectrum_matches_oracle():
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    gen = torch.Generator().manual_seed(64)
    x = torch.randn(1, 128, 128, 128, generator=gen)
    ref = O.so3_rfft(x, b_out=64)
    got = ops.so3_rfft(x.cuda(), b_out=64)
    assert_close(got, ref, "b=64 rfft")
    assert_close(ops.so3_rifft(got), O.so3_rifft(ref), "b=64 rifft")


@pytest.mark.gpu
@pytest.mark.parametrize("b_out", [64, 20])
def test_b64_plane_kernels_match_three_pass_path(b_out):
    """Every way the library can run 2b = 128 gives the same spectrum and signal (batch 11: a full
    chunk of 8 and a ragged one of 3; chunks of 2: five full and one of a single signal; b_out <
    b_in keeps a subset of columns)."""
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    gen = torch.Generator().manual_seed(66)
    x = torch.randn(11, 128, 128, 128, generator=gen).cuda()
    s = torch.randn(O.so3_nspec(b_out), 11, 2, generator=gen).cuda()
    res = {}
    try:
        for level, width in ((2, 0), (0, 0), (0, 2)):
            ops.lib.s2c_debug_force_general_path(level)
            ops.lib.s2c_debug_plane_chunk(width)
            res[(level, width)] = (ops.so3_rfft(x, b_out=b_out), ops.so3_rifft(s, b_out=64))
    finally:
        ops.lib.s2c_debug_force_general_path(0)
        ops.lib.s2c_debug_plane_chunk(0)
    ref_f, ref_i = res[(2, 0)]
    for key in ((0, 0), (0, 2)):
        assert_close(res[key][0], ref_f.cpu(), "rfft %s" % (key,))
        assert_close(res[key][1], ref_i.cpu(), "rifft %s" % (key,))


@pytest.mark.gpu
def test_b64_round_trip_properties():
    from s2cnn_b200.ops import cuda_ops
    ops = cuda_ops()
    gen = torch.Generator().manual_seed(65)
    x = torch.randn(6, 128, 128, 128, generator=gen).cuda()
    x1 = ops.so3_rifft(ops.so3_rfft(x))
    x2 = ops.so3_rifft(ops.so3_rfft(x1))
    assert ((x1 - x2).norm() / x2.norm()).item() < 1e-5          # idempotence
    a, b = x[:3], x[3:]
    lhs = ops.so3_rfft(2.0 * a - 0.5 * b)
    rhs = 2.0 * ops.so3_rfft(a) - 0.5 * ops.so3_rfft(b)
    assert ((lhs - rhs).norm() / rhs.norm()).item() < 1e-5        # linearity
