"""The tcgen05 / TMEM implementation of so3_mm (3xTF32) against the oracle, on shapes that
exercise: the benchmark layer (nl 6, batch 256, 20 -> 40), several K blocks per p (2 f_in > 48),
row tiles that straddle m, partial row and column tiles, and one degree only.  GPU only - the
kernel has no host emulation; the FP32 kernel it replaces is checked on both builds elsewhere."""
import pytest
import torch

from oracle import s2cnn_oracle as O
from util import assert_close

n3 = O.so3_nspec


@pytest.mark.gpu
@pytest.mark.parametrize("nl,nb,fi,fo", [(6, 256, 20, 40), (3, 130, 26, 6), (4, 100, 4, 64),
                                         (1, 1, 2, 2), (5, 3, 18, 2), (2, 300, 50, 10)])
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
