"""Test infrastructure (oracle side): import the UNMODIFIED reference CPU code path.

Only usable where a checkout of jonkhler/s2cnn is present (pass its path or set
``S2CNN_REFERENCE``) or where ``oracle/make_ref.py`` has left its untracked copy; it is used to
validate ``oracle/s2cnn_oracle.py``, to generate the golden fixtures under ``tests/golden/`` and by
the benchmark's CPU-baseline / reference arm to time the reference's own CPU code.  Neither the
product nor the GPU tests call this module.

The reference is seven years old; three shims are needed on a current stack, none of which
touches its arithmetic:

1. ``np.float`` alias (removed in numpy >= 1.24), used at s2cnn/s2_grid.py:10 and
   s2cnn/so3_grid.py:14.
2. ``torch.fft.rfftn`` called on a complex tensor at s2cnn/soft/so3_fft.py:94 (CPU branch
   of so3_rfft).  The loop below that line indexes negative ``n`` (:104-106), so the intent
   is the full complex spectrum; current torch raises instead.  The shim maps
   "rfftn of a complex tensor" to ``fftn`` and leaves real inputs alone.
3. The on-disk table cache writes ``./cache/...`` relative to the working directory
   (s2cnn/utils/decorator.py:68-70): we chdir into a scratch directory while importing and
   running.

``lie_learn`` (third party, absent, un-pinned) is replaced by the float64 restatement in
``oracle/wigner_np.py``.
"""
import contextlib
import os
import sys
import tempfile
import types

import numpy as np
import torch

from . import wigner_np

_DEFAULT_REF = os.environ.get("S2CNN_REFERENCE", "/root/reference")
_LOCAL_COPY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_state = {}


def local_copy():
    """Path of the untracked copy of the reference package made by ``oracle/make_ref.py`` (the form
    in which the reference travels to a machine without a checkout), or None."""
    return _LOCAL_COPY if os.path.isdir(os.path.join(_LOCAL_COPY, "s2cnn")) else None


def _install_lie_learn_standin():
    if "lie_learn" in sys.modules and getattr(sys.modules["lie_learn"], "_s2c_standin", False):
        return
    pkg = types.ModuleType("lie_learn")
    pkg._s2c_standin = True
    pkg.__path__ = []
    rep = types.ModuleType("lie_learn.representations")
    rep.__path__ = []
    so3 = types.ModuleType("lie_learn.representations.SO3")
    so3.__path__ = []
    wd = types.ModuleType("lie_learn.representations.SO3.wigner_d")
    wd.wigner_d_matrix = wigner_np.wigner_d_matrix
    wd.wigner_D_matrix = wigner_np.wigner_D_matrix
    spaces = types.ModuleType("lie_learn.spaces")
    spaces.__path__ = []
    s3 = types.ModuleType("lie_learn.spaces.S3")
    s3.quadrature_weights = wigner_np.quadrature_weights
    pkg.representations = rep
    rep.SO3 = so3
    so3.wigner_d = wd
    pkg.spaces = spaces
    spaces.S3 = s3
    for name, mod in [("lie_learn", pkg), ("lie_learn.representations", rep),
                      ("lie_learn.representations.SO3", so3),
                      ("lie_learn.representations.SO3.wigner_d", wd),
                      ("lie_learn.spaces", spaces), ("lie_learn.spaces.S3", s3)]:
        sys.modules[name] = mod


def _install_shims():
    if not hasattr(np, "float"):
        np.float = float  # shim 1
    if not getattr(torch.fft.rfftn, "_s2c_shim", False):
        real_rfftn = torch.fft.rfftn

        def rfftn(x, *args, **kwargs):  # shim 2
            if torch.is_complex(x):
                return torch.fft.fftn(x, *args, **kwargs)
            return real_rfftn(x, *args, **kwargs)

        rfftn._s2c_shim = True
        torch.fft.rfftn = rfftn


def available(path=None):
    path = path or _DEFAULT_REF
    return os.path.isdir(os.path.join(path, "s2cnn"))


def load(path=None):
    """Return the imported reference package ``s2cnn`` (cached)."""
    if "mod" in _state:
        return _state["mod"]
    path = path or _DEFAULT_REF
    if not available(path):
        raise RuntimeError("reference checkout not found at %r" % path)
    _install_lie_learn_standin()
    _install_shims()
    scratch = tempfile.mkdtemp(prefix="s2cnn_ref_cache_")
    _state["scratch"] = scratch
    sys.path.insert(0, path)
    sys.dont_write_bytecode = True
    try:
        with in_scratch():
            import s2cnn  # noqa: F401  (the reference)
            import s2cnn.soft.so3_fft  # noqa: F401
            import s2cnn.soft.s2_fft  # noqa: F401
    finally:
        sys.path.remove(path)
    _state["mod"] = sys.modules["s2cnn"]
    return _state["mod"]


@contextlib.contextmanager
def in_scratch():
    """Run a block with the working directory set to the scratch cache dir (shim 3)."""
    old = os.getcwd()
    os.chdir(_state["scratch"])
    try:
        with contextlib.redirect_stdout(open(os.devnull, "w")):
            yield
    finally:
        os.chdir(old)
