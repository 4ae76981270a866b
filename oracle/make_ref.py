"""Copies the `kvax/` package of a reference checkout to oracle/_ref/kvax_reference/ (ignored by git),
unmodified, so that oracle/triton_reference.py can run the reference's own Triton kernels on a GPU box
where the checkout itself is not mounted.  TEST / BENCH INFRASTRUCTURE ONLY.

    python -m oracle.make_ref /path/to/kvax-checkout
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "kvax_reference")


def make(ref_root: str) -> str:
    src = os.path.join(ref_root, "kvax")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src} is not a directory")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    shutil.copytree(src, os.path.join(DEST, "kvax"), ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    for extra in ("LICENSE", "README.md"):
        if os.path.exists(os.path.join(ref_root, extra)):
            shutil.copy(os.path.join(ref_root, extra), os.path.join(DEST, extra))
    return DEST


if __name__ == "__main__":
    print(make(sys.argv[1]))
