"""Every bandwidth of the single-kernel path (2b <= 32) against the library's own three separate
passes (an independent implementation, itself pinned to the oracle by the other tests), with batch
sizes that are not multiples of the four signals a block owns: analysis (both weightings, ReLU on
load, with the per-signal sums), synthesis (both weightings, with the ReLU mask on store) and the
complex synthesis.  About 1800 comparisons; float32, relative L2 error below 2e-5."""
import random

import pytest
import torch


def _rel(a, b):
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


@pytest.mark.gpu
def test_single_kernel_paths_match_three_pass_path_for_every_bandwidth():
    from s2cnn_b200.ops import cuda_ops, so3_nspec
    ops = cuda_ops()
    lib = ops.lib
    rng = random.Random(0)
    torch.manual_seed(0)
    worst = {}
    try:
        for b_in in range(1, 17):
            for b_out in sorted({1, 2, 3, 5, 6, 8, 10, 12, 13, 14, 15, 16, b_in}):
                nb = rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 13])
                x = torch.randn(nb, 2 * b_in, 2 * b_in, 2 * b_in, device="cuda")
                s = torch.randn(so3_nspec(b_in), nb, 2, device="cuda")
                act = torch.randn(nb, 2 * b_out, 2 * b_out, 2 * b_out, device="cuda")
                res = {}
                for level in (0, 2):
                    lib.s2c_debug_force_general_path(level)
                    res[level] = dict(
                        rfft=ops.so3_rfft(x, b_out=b_out),
                        rfft_grad=ops.so3_rfft(x, for_grad=True, b_out=b_out),
                        rifft=ops.so3_rifft(s, b_out=b_out),
                        rifft_grad=ops.so3_rifft(s, for_grad=True, b_out=b_out),
                        ifft=ops.so3_ifft(s, b_out=b_out))
                res[2]["relu"] = ops.so3_rfft(torch.relu(x), b_out=b_out)
                res[2]["sums_spectrum"] = res[2]["rfft_grad"]
                res[2]["sums"] = x.double().sum(dim=(-3, -2, -1)).float()
                res[2]["mask"] = res[2]["rifft_grad"] * (act > 0)
                lib.s2c_debug_force_general_path(0)
                res[0]["relu"] = ops.so3_rfft(x, b_out=b_out, relu=True)
                res[0]["sums_spectrum"], res[0]["sums"] = ops.so3_rfft_with_sums(x, for_grad=True,
                                                                                 b_out=b_out)
                res[0]["mask"] = ops.so3_rifft_relu_grad(s, act)
                for k in res[0]:
                    e = _rel(res[0][k], res[2][k])
                    if e > worst.get(k, (0.0,))[0]:
                        worst[k] = (e, b_in, b_out, nb)
    finally:
        lib.s2c_debug_force_general_path(0)
    bad = {k: v for k, v in worst.items() if not v[0] < 2e-5}
    assert not bad, "worst (rel-L2, b_in, b_out, batch) per op: %r" % (worst,)
