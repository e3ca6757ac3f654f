"""Put the reference's own attention package where the benchmark can import it.

    python oracle/make_ref.py --ref /path/to/reference

Copies the reference's ``ma/`` package (pure Python: the module API, the eager implementation and
the Triton implementation) unmodified into ``oracle/_ref/ma/``.  ``oracle/_ref/`` is git-ignored -
reference sources are never committed - but it travels with the working tree, so that
``bench.py`` can time the reference's GPU paths (eager PyTorch on the GPU, Triton) next to this
library on the same device.  Test infrastructure only: nothing in the product imports it.
"""
from __future__ import annotations

import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(ref: str) -> str | None:
    src = os.path.join(ref, "ma")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "ma")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "tests"))
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference repository")
    print(make_ref(ap.parse_args().ref))
