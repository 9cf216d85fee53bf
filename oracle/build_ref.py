"""Installs the UNMODIFIED reference package next to the oracle, as the thing the oracle is checked against.

    python oracle/build_ref.py [--reference /path/to/tt-boltz]

Test infrastructure: only ``tests/``, ``__graft_entry__`` and the CPU legs of ``bench.py`` may use what this
writes.  The reference is pure Python; "building" it is an offline ``pip install --no-deps --target oracle/_ref``
of its checkout (from a scratch copy, because a read-only checkout cannot hold the build's egg-info).  Nothing
is copied into the tracked tree: ``oracle/_ref/`` is git-ignored.  Its one missing import, the ``ttnn`` device
library, is stubbed at import time by ``oracle/ref_modules.py``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def default_reference() -> str:
    """$TT_BIO_REFERENCE, else a checkout called ``reference`` beside this repository."""
    return os.environ.get("TT_BIO_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference: str | None = None, force: bool = False) -> str | None:
    """Returns the install directory, or None when no reference checkout is present (then whatever was
    installed earlier, if anything, stays in use)."""
    reference = reference or default_reference()
    if not os.path.isdir(os.path.join(reference, "tt_bio")):
        return TARGET if os.path.isdir(os.path.join(TARGET, "tt_bio")) else None
    if os.path.isdir(os.path.join(TARGET, "tt_bio")) and not force:
        return TARGET
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "src")
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns(".git", "examples", "docs"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
               "--target", TARGET, "--upgrade", src]
        if os.environ.get("PIP_FIND_LINKS"):          # an offline wheel folder, if the environment names one
            cmd[5:5] = ["--find-links", os.environ["PIP_FIND_LINKS"]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("pip install of the reference failed")
    return TARGET


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
