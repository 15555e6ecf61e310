"""The allocation-free synthesis entry point, s2c_so3_rifft_static.

It exists for callers that cannot get device memory when they call the library - a process whose
GPU is entirely pre-reserved by another allocator, or a loop that must not pay the device-wide
synchronisation of cudaMalloc / cudaFree - and therefore keeps its scratch and tables in static
device arrays inside the library.  The test calls it through the C ABI several times in a row
(a repeat with the tables already loaded, then other data, a bias and the other table weighting, so
stale scratch or tables would show) and compares each result with the regular entry point
s2c_so3_rifft on the same inputs and with the CPU oracle, at the suite's tolerance (relative L2 <=
1e-4).  On the CUDA build the regular entry point takes the single-kernel path at these sizes while
the static one runs the three separate passes, so the comparison is between two implementations;
both are float32 sums in different orders and agree to a few 1e-7.  It also checks that both size
limits (scratch bytes, table bytes) are enforced with an error.  The file name sorts last on
purpose: if it fails, every other test has already run.
"""
import pytest
import torch

import backends
from util import assert_close


def n3(b):
    return b * (4 * b * b - 1) // 3


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_static_entry_point_matches_regular_one_twice(backend):
    ops, dev = backends.get(backend)
    lib = ops.lib
    stream = torch.cuda.current_stream().cuda_stream if dev.type == "cuda" else None
    gen = torch.Generator().manual_seed(2024)
    from oracle import s2cnn_oracle as O
    cases = [
        # (b_in, b_out, nbatch, for_grad, with_bias)
        (6, 6, 12, 0, False),
        (6, 6, 12, 0, False),   # same configuration again: tables already in the static array
        (6, 4, 10, 1, True),
        (6, 6, 12, 0, False),   # back to the first configuration: tables reloaded
    ]
    for b_in, b_out, nb, fg, with_bias in cases:
        x = torch.randn(n3(b_in), nb, 2, generator=gen).to(dev)
        bias = torch.randn(5, generator=gen).to(dev) if with_bias else None
        n = 2 * b_out
        ref = torch.empty(nb, n, n, n, device=dev)
        ws = torch.empty(lib.s2c_so3_fft_workspace(nb, b_in, b_out), dtype=torch.uint8, device=dev)
        lib.call("s2c_so3_rifft", x.data_ptr(), ref.data_ptr(), nb, b_in, b_out, fg,
                 bias.data_ptr() if with_bias else None, 5 if with_bias else 0,
                 ws.data_ptr(), ws.numel(), stream)
        out = torch.full((nb, n, n, n), float("nan"), device=dev)
        lib.call("s2c_so3_rifft_static", x.data_ptr(), out.data_ptr(), nb, b_in, b_out, fg,
                 bias.data_ptr() if with_bias else None, 5 if with_bias else 0, stream)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        assert not torch.isnan(out).any()
        assert_close(out, ref, "static vs regular (b %d->%d)" % (b_in, b_out))
        want = O.so3_rifft(x.cpu(), for_grad=bool(fg), b_out=b_out)
        if with_bias:
            want = want + bias.cpu().repeat(nb // 5).view(nb, 1, 1, 1)
        assert_close(out, want, "static vs oracle (b %d->%d)" % (b_in, b_out))


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_static_entry_point_rejects_oversized_calls(backend):
    ops, dev = backends.get(backend)
    lib = ops.lib
    limit = lib.s2c_so3_rifft_static_max_bytes()
    b = 8
    per = lib.s2c_so3_fft_workspace_min(b, b)
    nb = limit // per + 1
    x = torch.zeros(16, device=dev)  # never read: the size check comes first
    rc = lib.s2c_so3_rifft_static(x.data_ptr(), x.data_ptr(), nb, b, b, 0, None, 0, None)
    assert rc != 0
    assert "static array holds" in lib.last_error()


@pytest.mark.parametrize("backend", backends.BACKENDS)
def test_static_entry_point_rejects_tables_beyond_the_static_array(backend):
    """b = 32 needs about 5.6 MB of Wigner tables, more than the 4 MiB static table array: the call
    must fail with a message instead of overrunning the array (the scratch check passes: one signal
    of 64^3 needs 2 MB of the 32 MiB)."""
    ops, dev = backends.get(backend)
    lib = ops.lib
    b = 32
    assert lib.s2c_so3_fft_workspace_min(b, b) <= lib.s2c_so3_rifft_static_max_bytes()
    x = torch.zeros(16, device=dev)  # never read: the table check comes before any launch
    rc = lib.s2c_so3_rifft_static(x.data_ptr(), x.data_ptr(), 1, b, b, 0, None, 0, None)
    assert rc != 0
    assert "static table array holds" in lib.last_error()
    # ... and the entry point still works afterwards
    nb, bb = 4, 5
    gen = torch.Generator().manual_seed(5)
    xs = torch.randn(n3(bb), nb, 2, generator=gen).to(dev)
    out = torch.empty(nb, 2 * bb, 2 * bb, 2 * bb, device=dev)
    stream = torch.cuda.current_stream().cuda_stream if dev.type == "cuda" else None
    lib.call("s2c_so3_rifft_static", xs.data_ptr(), out.data_ptr(), nb, bb, bb, 0, None, 0, stream)
    from oracle import s2cnn_oracle as O
    assert_close(out, O.so3_rifft(xs.cpu()), "static entry point after a rejected call")
