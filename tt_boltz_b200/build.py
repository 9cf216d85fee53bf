"""Ahead-of-time build of libb200pf.so (sm_100a only) with plain nvcc.

    python -m tt_boltz_b200.build [--force] [--verbose]

Objects and the shared library are written next to the sources (``csrc/_build``,
``tt_boltz_b200/libb200pf.so``); both are git-ignored build artefacts.  nvcc cross-compiles
without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(CSRC, "_build")
LIB = os.path.join(PKG, "libb200pf.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-DB200PF_BUILD",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the b200pf kernels cannot be built")


def have_nvcc() -> bool:
    try:
        _nvcc()
        return True
    except RuntimeError:
        return False


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stamp() -> str:
    """Hash of every source and header (by name relative to the package, so that a copy of the tree elsewhere
    keeps its stamp) and of the compiler flags."""
    h = hashlib.sha256()
    files = sources() + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    files.append(os.path.join(INCLUDE, "b200pf.h"))
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _up_to_date(stamp: str) -> bool:
    stamp_file = os.path.join(OUT, "stamp")
    return os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    stamp = _stamp()
    if not force and _up_to_date(stamp):
        return LIB
    # Several processes may get here at once (one rank per GPU): one builds, the others wait for the lock and
    # then find the library up to date.  The library is linked under a temporary name and renamed into place,
    # so nobody ever loads a half-written file.
    import fcntl
    with open(os.path.join(OUT, "lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and _up_to_date(stamp):
            return LIB
        nvcc = _nvcc()
        extra = ["-Xptxas", "-v"] if verbose else []

        def compile_one(src: str) -> str:
            obj = os.path.join(OUT, os.path.basename(src)[:-3] + ".o")
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", INCLUDE, "-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, sources()))
        tmp = LIB + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libb200pf.so failed")
        os.replace(tmp, LIB)
        with open(os.path.join(OUT, "stamp"), "w") as fh:
            fh.write(stamp)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
