"""Bandwidth 64 (the standalone-FFT benchmark size, 2b = 128 -> two-step 8 x 16 register FFT) on
the GPU: spectrum parity against the oracle for one batch element, the reference's idempotence
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
