"""Small, fixed workloads for profiler captures of single kernels.

    python -m s2cnn_b200._profile_cases <case>

Each case runs one op a few times on seeded synthetic data sized for a capture that ends by itself
within a minute (inputs above the 126 MB L2 where DRAM figures matter, a few hundred MB at most):

    inv10   so3_rifft, b = 10, 5120 signals          (kernel so3_inv_fused<20>)
    fwd10   so3_rfft,  b = 10 -> 6, 5120 signals     (kernel so3_fwd_fused<20>)
    inv16   so3_rifft, b = 16, 1600 signals          (kernel so3_inv_fused<32>, 512-thread blocks)
    fwd16   so3_rfft,  b = 16, 1600 signals          (kernel so3_fwd_fused<32>, 512-thread blocks)
    relay10 s2_mm + so3_rifft (b = 10) + bias + ReLU + so3_rfft (-> b = 6), batch 256, 1 -> 20
            features = 5120 signals                  (kernel so3_relay_fused<20>)
    mm      so3_mm, nl = 6, batch 256, 20 -> 40      (kernel so3_mm_tc_kernel)
    mm_c4   so3_mm, nl = 10, batch 32, 100 -> 100    (kernel so3_mm_tc_kernel at a GEMM-sized case)
    fft64   so3_rfft + so3_rifft, b = 64, 8 signals  (plane kernels + Wigner contraction)
    fft64_three_pass   the same through the three separate passes (the path 2b = 256 takes)
"""
import sys

import torch

from .ops import cuda_ops, so3_nspec


def main(which):
    ops = cuda_ops()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    if which == "inv10":
        s = torch.randn(so3_nspec(10), 5120, 2, device=dev)
        for _ in range(3):
            ops.so3_rifft(s)
    elif which == "fwd10":
        x = torch.randn(5120, 20, 20, 20, device=dev)
        for _ in range(3):
            ops.so3_rfft(x, b_out=6)
    elif which == "inv16":
        s = torch.randn(so3_nspec(16), 1600, 2, device=dev)
        for _ in range(3):
            ops.so3_rifft(s)
    elif which == "fwd16":
        x = torch.randn(1600, 32, 32, 32, device=dev)
        for _ in range(3):
            ops.so3_rfft(x)
    elif which == "relay10":
        xs = torch.randn(100, 256, 1, 2, device=dev)
        ys = torch.randn(100, 1, 20, 2, device=dev)
        bias = torch.randn(20, device=dev)
        for _ in range(3):
            ops.s2_conv_relu_so3_rfft(xs, ys, bias, 6)
    elif which == "mm":
        x = torch.randn(so3_nspec(6), 256, 20, 2, device=dev)
        y = torch.randn(so3_nspec(6), 20, 40, 2, device=dev)
        for _ in range(3):
            ops.so3_mm(x, y)
    elif which == "mm_c4":
        x = torch.randn(so3_nspec(10), 32, 100, 2, device=dev)
        y = torch.randn(so3_nspec(10), 100, 100, 2, device=dev)
        for _ in range(3):
            ops.so3_mm(x, y)
    elif which in ("fft64", "fft64_three_pass"):
        x = torch.randn(8, 128, 128, 128, device=dev)
        ops.lib.s2c_debug_force_general_path(2 if which == "fft64_three_pass" else 0)
        for _ in range(2):
            ops.so3_rifft(ops.so3_rfft(x))
        ops.lib.s2c_debug_force_general_path(0)
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "")
