"""Stages the reference's own Python package for the CPU baseline of the benchmark.

    python oracle/stage_reference.py [/path/to/reference/checkout]

The reference (NeuroMarshal/bitlattice) runs its hot path on the CPU with PyTorch alone when its CUDA extension is
absent (``bitlattice/_ops.py`` falls back to ``bitlattice/reference.py``). This script copies the Python files of its
``bitlattice`` package, unmodified, from the read-only checkout into ``oracle/_ref/bitlattice`` -- a build output that
is never committed -- so that ``bench.py --impl reference`` can drive the reference itself (``F.linear`` on the exact
route, ``bitlattice.optim.Lattice(...).step()``) on a machine that has no checkout. Without the checkout nothing is
staged and the benchmark times the C restatement (``oracle/bl_oracle.c``) instead.

Test infrastructure: nothing in the product imports what this stages.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SOURCE = "/root/reference"


def stage(source: str = DEFAULT_SOURCE) -> str | None:
    """Copy ``<source>/bitlattice/**/*.py`` to ``oracle/_ref/bitlattice``; returns the destination, or None when the
    checkout is absent."""
    pkg = os.path.join(source, "bitlattice")
    if not os.path.isdir(pkg):
        return None
    dest = os.path.join(DEST, "bitlattice")
    if os.path.isdir(dest):
        shutil.rmtree(dest)
    shutil.copytree(pkg, dest, ignore=lambda d, names: [n for n in names if n == "__pycache__" or
                                                         (os.path.isfile(os.path.join(d, n)) and not n.endswith(".py"))])
    with open(os.path.join(DEST, "SOURCE"), "w") as f:
        f.write(f"unmodified copy of {pkg} (Python files only)\n")
    return dest


def staged_path() -> str | None:
    """``oracle/_ref`` when a staged package exists there."""
    return DEST if os.path.isfile(os.path.join(DEST, "bitlattice", "__init__.py")) else None


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SOURCE)
    print(out or "no reference checkout: nothing staged")
