"""Test infrastructure: make a local, untracked copy of the reference's Python package.

    python -m oracle.make_ref [path-to-reference-checkout]

The reference (jonkhler/s2cnn) is pure Python, so "building" it for the CPU baseline means having
its package importable where the benchmark runs.  This copies ``<checkout>/s2cnn`` - unmodified -
to ``oracle/_ref/s2cnn``.  The directory is listed in .gitignore: it is a build artefact like a
compiled reference would be, never part of the history.  ``bench.py --impl reference`` and the
``cpu_baseline`` leg time that copy when it exists (``kind: "reference"``) and fall back to the
oracle port otherwise.  Nothing in the product imports it.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make(src="/root/reference"):
    pkg = os.path.join(src, "s2cnn")
    if not os.path.isdir(pkg):
        return None
    out = os.path.join(DEST, "s2cnn")
    if os.path.isdir(out):
        shutil.rmtree(out)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(pkg, out, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.pdf"))
    return DEST


if __name__ == "__main__":
    print(make(*(sys.argv[1:2])))
