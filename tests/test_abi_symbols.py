"""The shared library must load on a CPU-only machine and export every function that
include/b200pf.h declares (no compute calls here)."""
import ctypes
import os
import re

from tt_boltz_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200pf.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200pf_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_all_declared_symbols():
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in b200pf.h but not exported"


def test_binding_covers_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_version_and_error_string_without_gpu():
    lib = _lib.load()
    assert lib.b200pf_version() >= 100
    assert isinstance(_lib.last_error(), str)
    # argument validation happens before any CUDA call
    rc = lib.b200pf_f32_layernorm(None, None, None, None, 4, 128, None)
    assert rc == -1 and "bad argument" in _lib.last_error()
