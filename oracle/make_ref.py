"""Places the reference's own Python package under ``oracle/_ref/`` (git-ignored).

    python oracle/make_ref.py /path/to/reference      (or FLASHQUANT_REFERENCE_ROOT=...)

The reference (ayinedjimi/flashquant) is pure Python on its CPU path, so "building" it is a
copy of ``src/flashquant`` as it lies in the checkout.  The copy is test and benchmark
infrastructure only: ``bench.py --impl reference`` times the reference's own
``flashquant.kernels.paged_decode.split_k_paged_decode`` (CPU branch) from it when it is there
and falls back to the oracle restatement otherwise.  Nothing in the product package imports it,
and it is never committed.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(reference_root: str | None = None) -> str | None:
    reference_root = reference_root or os.environ.get("FLASHQUANT_REFERENCE_ROOT", "")
    src = os.path.join(reference_root, "src", "flashquant")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "flashquant")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so"))
    return dst


if __name__ == "__main__":
    out = make_ref(*sys.argv[1:2])
    print(out if out else "no reference checkout found: nothing copied")
