"""Mirrors the few reference files the hot path's drop-in checks and the same-box comparison need into
baseline/_ref/ (git-ignored: the reference is never part of this repository's history).

The reference is a source tree without an installable package, so "installing" it means placing its modules where a
test or the benchmark can import them on a machine that has no reference checkout of its own: the port model
`looped_transformer.py` with the readers it imports, the Triton module `fused_dattn.py`, and the trainer model's package
`trainer/flame/custom_models/`. Files are copied byte for byte, never edited.

    python baseline/stage_reference.py [reference root]      (default: $LOOPBACK_REF, else DEFAULT_ROOT below)
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ("looped_transformer.py", "loop_linattn_state.py", "loop_linattn_delta.py", "fused_dattn.py", "LICENSE",
         os.path.join("trainer", "flame", "__init__.py"))
TREES = (os.path.join("trainer", "flame", "custom_models"),)
DEFAULT_ROOT = os.path.join(os.sep, "root", "reference")     # where the build machine keeps its reference checkout


def default_source() -> str | None:
    for cand in (os.environ.get("LOOPBACK_REF"), DEFAULT_ROOT):
        if cand and os.path.isfile(os.path.join(cand, "fused_dattn.py")):
            return cand
    return None


def stage(src: str | None = None) -> str | None:
    """Copy the files; returns the destination, or None when no reference checkout is reachable (then an
    existing baseline/_ref/ is left as it is)."""
    src = src or default_source()
    if src is None:
        return DEST if os.path.isdir(DEST) else None
    for rel in FILES:
        s = os.path.join(src, rel)
        if os.path.isfile(s):
            os.makedirs(os.path.dirname(os.path.join(DEST, rel)), exist_ok=True)
            shutil.copyfile(s, os.path.join(DEST, rel))
    for rel in TREES:
        s = os.path.join(src, rel)
        if os.path.isdir(s):
            shutil.copytree(s, os.path.join(DEST, rel), dirs_exist_ok=True,
                            ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


def find() -> str | None:
    """Where a reference tree can be imported from at run time: $LOOPBACK_REF, else baseline/_ref/."""
    for cand in (os.environ.get("LOOPBACK_REF"), DEST):
        if cand and os.path.isfile(os.path.join(cand, "fused_dattn.py")):
            return cand
    return None


if __name__ == "__main__":
    print(stage(sys.argv[1] if len(sys.argv) > 1 else None))
