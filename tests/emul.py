"""Host-emulation build of the kernel sources for the CPU test-suite.

The library's single translation unit is compiled with g++ and -DS2C_EMUL: CUDA threads run as
fibers, barriers as fiber switches.  Test infrastructure only - nothing in the product loads it.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC_DIR = os.path.join(ROOT, "s2cnn_b200", "csrc")
OUT_DIR = os.path.join(HERE, "_emul")
OUT = os.path.join(OUT_DIR, "libs2cnn_emul.so")

_ops = None


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    srcs = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR)]
    srcs.append(os.path.join(ROOT, "include", "s2cnn_b200.h"))
    return any(os.path.getmtime(s) > t for s in srcs)


def build():
    if _stale():
        os.makedirs(OUT_DIR, exist_ok=True)
        cmd = ["g++", "-x", "c++", "-std=c++17", "-O2", "-DS2C_EMUL", "-fPIC", "-shared", "-o",
               OUT, os.path.join(SRC_DIR, "lib.cu")]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError("emulation build failed:\n" + res.stdout)
    return OUT


def ops():
    """An ``Ops`` bound to the emulation build (CPU tensors)."""
    global _ops
    if _ops is None:
        from s2cnn_b200 import _lib
        from s2cnn_b200.ops import Ops
        _ops = Ops(_lib.Lib(build()))
    return _ops
