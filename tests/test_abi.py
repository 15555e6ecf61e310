"""The C-ABI boundary itself: the CUDA library builds, loads without a GPU, exports every symbol
that include/s2cnn_b200.h declares, and reports errors as status codes with a message.  No device
computation is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from s2cnn_b200 import _lib, build as build_mod

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cuda_lib():
    build_mod.build()
    return _lib.Lib(_lib.CUDA_LIB_PATH)


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "s2cnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(s2c_\w+)\s*\(", text)))


def test_header_and_binding_agree(cuda_lib):
    declared = _declared_symbols()
    assert len(declared) >= 30
    assert set(declared) == set(_lib.EXPORTED_SYMBOLS)
    raw = ctypes.CDLL(_lib.CUDA_LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert cuda_lib.s2c_is_cuda_build() == 1
    assert cuda_lib.s2c_version() >= 100


def test_host_generators_need_no_gpu(cuda_lib):
    from oracle import wigner_np
    for l, beta in [(0, 0.3), (1, 0.37), (4, 2.9), (31, 1.234), (63, 0.01)]:
        out = np.empty((2 * l + 1, 2 * l + 1))
        cuda_lib.call("s2c_wigner_d", l, beta, out.ctypes.data)
        assert np.abs(out - wigner_np.wigner_d_matrix(l, beta)).max() < 1e-12
    out = np.empty((3, 3))
    cuda_lib.call("s2c_wigner_d", 1, 0.5, out.ctypes.data)
    assert abs(out[1, 1] - np.cos(0.5)) < 1e-15 and abs(out[2, 1] + np.sin(0.5) / np.sqrt(2)) < 1e-15
    for b in (1, 2, 7, 64):
        w = np.empty(2 * b)
        cuda_lib.call("s2c_quadrature_weights", b, w.ctypes.data)
        assert np.abs(w - wigner_np.quadrature_weights(b)).max() < 1e-17
        assert abs(w.sum() * (2 * b) ** 2 - 1) < 1e-13


def test_tables_in_reference_layout_match_golden(cuda_lib):
    from util import golden
    g = golden("tables")
    for key, (b, nl, w, s2) in {"so3_5_4_w": (5, 4, 1, False), "so3_5_4_u": (5, 4, 0, False),
                                "so3_3_6_w": (3, 6, 1, False), "s2_6_5_w": (6, 5, 1, True),
                                "s2_6_5_u": (6, 5, 0, True)}.items():
        ref = g[key].float().numpy()
        out = np.empty(ref.shape, dtype=np.float32)
        cuda_lib.call("s2c_s2_wigner_table" if s2 else "s2c_so3_wigner_table", b, nl, w, out.ctypes.data)
        assert np.abs(out - ref).max() <= 1e-7 * max(1.0, np.abs(ref).max()), key


def test_wigner_symmetries():
    """Identities the kernels rely on (mirror rows of real signals)."""
    from oracle import wigner_np
    lib = _lib.Lib(_lib.CUDA_LIB_PATH)
    l, beta = 6, 0.83
    d = np.empty((13, 13))
    lib.call("s2c_wigner_d", l, beta, d.ctypes.data)
    m = np.arange(-l, l + 1)
    sign = (-1.0) ** (m[:, None] - m[None, :])
    assert np.abs(d[::-1, ::-1] - sign * d).max() < 1e-13          # d_{-m,-n} = (-1)^(m-n) d_{mn}
    assert np.abs(d.T - sign * d).max() < 1e-13                    # d_{nm} = (-1)^(m-n) d_{mn}
    assert np.abs(d @ d.T - np.eye(13)).max() < 1e-13              # orthogonal


def test_errors_are_status_codes(cuda_lib):
    rc = cuda_lib.s2c_so3_rfft(None, None, 1, 4, 4, 0, None, 0, None)
    assert rc != 0 and "bad argument" in cuda_lib.last_error()
    rc = cuda_lib.s2c_s2_fft(ctypes.c_void_p(16), 1, ctypes.c_void_p(16), 1, 3, 5, 0, None, 0, None)
    assert rc != 0 and "b_out <= b_in" in cuda_lib.last_error()
    rc = cuda_lib.s2c_so3_mm(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 0, 1, 1, 1, None)
    assert rc != 0
    with pytest.raises(_lib.S2cError):
        cuda_lib.call("s2c_quadrature_weights", 0, None)
    assert cuda_lib.s2c_so3_fft_workspace_min(4, 4) == (4 * 8 * 8 + 4 * 7 * 8) * 8
    assert cuda_lib.s2c_so3_fft_workspace(1000, 10, 6) >= 32 * cuda_lib.s2c_so3_fft_workspace_min(10, 6)


def test_product_refuses_cpu_tensors():
    """No CPU fallback: the public API bound to the CUDA build rejects host tensors loudly."""
    import s2cnn_b200
    from s2cnn_b200.soft.so3_fft import so3_rfft
    with pytest.raises(_lib.S2cError):
        so3_rfft(torch.zeros(4, 4, 4))
    with pytest.raises(_lib.S2cError):
        s2cnn_b200.so3_mm(torch.zeros(1, 1, 1, 2), torch.zeros(1, 1, 1, 2))


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(_lib.S2cError):
        _lib.Lib(str(tmp_path / "nope.so"))
