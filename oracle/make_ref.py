"""Places the UNMODIFIED reference package under `oracle/_ref/` (git-ignored) so that the
benchmark's reference arm and the tests can import `float8_experimental` itself on machines where
the reference checkout is not mounted.  TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing in the
product package imports it.

    python oracle/make_ref.py [path-to-reference-checkout]        (default: REFERENCE_ROOT below)

The reference is pure Python (no native code to compile) and declares `hatchling` as its build
backend, which an offline `pip install --no-index` cannot satisfy; the recipe therefore copies the
package directory `float8_experimental/` as it is.  No file is edited; nothing but that directory
is written, and only below `oracle/_ref/`.  Returns / prints the destination, or None when the
checkout is absent (the callers then fall back to the CPU restatement in `oracle/`).
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PACKAGE = "float8_experimental"
REFERENCE_ROOT = os.environ.get("F8_REFERENCE_ROOT", "/root/reference")  # where the build machine mounts the checkout


def make_ref(reference_root: str = REFERENCE_ROOT):
    src = os.path.join(reference_root, PACKAGE)
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, PACKAGE)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


def ref_path():
    """`oracle/_ref` when the reference package is there, else None."""
    return DEST if os.path.isfile(os.path.join(DEST, PACKAGE, "__init__.py")) else None


if __name__ == "__main__":
    print(make_ref(*sys.argv[1:2]))
