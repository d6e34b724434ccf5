"""Stage the reference's own kernel files for the checker.  Test infrastructure only.

    python -m oracle.make_ref [--root <reference checkout>]

Copies, unmodified, the six files of ``mdy_triton/core/`` that hold the reference's Triton kernels and
their autograd wrappers into ``oracle/_ref/`` (a git-ignored folder: the files never enter this
repository's history).  From there ``oracle/ref_loader.py`` loads them one by one

  * on a machine without a GPU under Triton's interpreter (golden vectors, oracle pinning), and
  * on a GPU natively through Triton's JIT, which is how the GPU parity tests and the benchmark's
    ``triton_reference`` leg run the reference's kernels on the same device as this library's.

The checkout is looked for in ``--root``, then ``MDY_REFERENCE_ROOT``, then a ``reference`` directory
beside this repository.  Nothing here is imported by the product package.
"""
from __future__ import annotations

import argparse
import os
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
FILES = ("rmsnorm.py", "fused_add_norm.py", "fused_apply_rope.py", "fused_silu.py", "cross_entyopy_loss.py",
         "triton_maxmin.py")


def find_checkout(root: str | None = None) -> Path | None:
    """The reference checkout's root, or None."""
    for cand in (root, os.environ.get("MDY_REFERENCE_ROOT"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "mdy_triton" / "core" / FILES[0]).exists():
            return Path(cand)
    return None


def stage(root: str | None = None, quiet: bool = False) -> bool:
    """Copy the kernel files into ``oracle/_ref/`` when a checkout is found.  Returns whether the folder
    holds all of them afterwards (a machine without the checkout keeps what was staged earlier)."""
    src_root = find_checkout(root)
    if src_root is not None:
        DEST.mkdir(exist_ok=True)
        for f in FILES:
            src = src_root / "mdy_triton" / "core" / f
            dst = DEST / f
            if not dst.exists() or dst.read_bytes() != src.read_bytes():
                shutil.copyfile(src, dst)
        if not quiet:
            print(f"staged {len(FILES)} reference kernel files from {src_root} into {DEST}")
    elif not quiet:
        print("no reference checkout found; keeping what is staged")
    return all((DEST / f).exists() for f in FILES)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", default=None)
    a = ap.parse_args()
    raise SystemExit(0 if stage(a.root) else 1)
