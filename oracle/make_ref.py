"""Vendors the reference for timing and fixture generation. TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [/path/to/sparsify-checkout]

Copies the `sparsify/` package directory of a checkout of EleutherAI/sparsify
v1.3.0 (the argument, else $SPARSIFY_REF) into `oracle/_ref/sparsify/`,
unmodified. `oracle/_ref/` is git-ignored - the reference's sources never enter this
repository's history - but it sits inside the working tree, so it is present
wherever the tree is copied to after this script ran (like the compiled kernel
library). `oracle/ref_loader.py` imports it from there.
"""

from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def make_ref(src: str | os.PathLike | None = None, quiet: bool = False) -> Path | None:
    candidates = [src, os.environ.get("SPARSIFY_REF")]
    root = next((Path(c) for c in candidates if c and Path(c, "sparsify", "fused_encoder.py").exists()), None)
    if root is None:
        if not quiet:
            print("make_ref: no reference checkout found (argument or $SPARSIFY_REF)", file=sys.stderr)
        return DEST if (DEST / "sparsify" / "fused_encoder.py").exists() else None
    target = DEST / "sparsify"
    DEST.mkdir(exist_ok=True)
    if target.exists():
        shutil.rmtree(target)
    shutil.copytree(root / "sparsify", target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    for extra in ("LICENSE", "pyproject.toml"):
        if (root / extra).exists():
            shutil.copy2(root / extra, DEST / extra)
    if not quiet:
        print(f"make_ref: copied {root / 'sparsify'} -> {target}")
    return DEST


if __name__ == "__main__":
    out = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    sys.exit(0 if out is not None else 1)
