"""Stage the reference's operator sources for machines that do not have its checkout.

    python oracle/make_ref.py [<reference root>]

TEST / BENCHMARK INFRASTRUCTURE ONLY.  Copies ``<reference root>/operators/*.py`` unmodified into
``oracle/_ref/operators/`` (a directory that is kept out of version control) and writes a
``MANIFEST`` with the sha256 of every file.  ``oracle/ref_loader.py`` imports the reference from
there when the checkout itself is absent, so that

  * ``bench.py --impl reference`` can time the reference's own
    ``true_divide_outlier_suboutlier_svd_compress`` (operators/compress_function.py:136-200) on the
    benchmark machine's host cores, and
  * the GPU parity tests can run the reference's forward norm kernels
    (operators/efficient_rmsnorm.py:15-60, operators/efficient_layernorm.py:15-62) beside this
    library's.

Nothing in the shipped package reads that directory.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_root() -> str:
    return os.environ.get("HYC_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def make(root: str | None = None) -> bool:
    """Returns True when ``oracle/_ref`` holds a copy afterwards (fresh or already there)."""
    root = root or default_root()
    src = os.path.join(root, "operators")
    if not os.path.isdir(src):
        return os.path.isdir(os.path.join(DEST, "operators"))
    dst = os.path.join(DEST, "operators")
    os.makedirs(dst, exist_ok=True)
    lines = []
    for name in sorted(os.listdir(src)):
        if not name.endswith(".py"):
            continue
        shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
        lines.append(f"{hashlib.sha256(open(os.path.join(dst, name), 'rb').read()).hexdigest()}  operators/{name}")
    with open(os.path.join(DEST, "MANIFEST"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return True


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else None)
    print("oracle/_ref ready" if ok else "reference checkout not found; nothing staged")
