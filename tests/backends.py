"""Test parametrisation over the two builds of the same kernel sources:

* ``"emul"`` - host-emulation build (CPU tensors); runs everywhere, exercises kernel bodies,
  index arithmetic, dispatch and table builders without a GPU;
* ``"cuda"`` - the product library on ``cuda:0`` (marked ``gpu``).

``active(backend)`` temporarily points the package's op table at the chosen build so that the
public API (functions, autograd rules, modules) can be driven on either.
"""
import contextlib

import pytest
import torch

BACKENDS = [pytest.param("emul"), pytest.param("cuda", marks=pytest.mark.gpu)]


def get(backend):
    if backend == "emul":
        import emul
        return emul.ops(), torch.device("cpu")
    from s2cnn_b200 import _lib
    from s2cnn_b200.ops import Ops
    return Ops(_lib.cuda_lib()), torch.device("cuda:0")


@contextlib.contextmanager
def active(backend):
    from s2cnn_b200 import ops as ops_mod
    o, dev = get(backend)
    old = ops_mod._cuda_ops
    ops_mod._cuda_ops = o
    try:
        yield o, dev
    finally:
        ops_mod._cuda_ops = old
