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


def test_msa_entry_points_validate_before_any_cuda_call():
    """Null pointers, token counts that do not fit the padded axis, misaligned groups: refused with a message, no launch."""
    lib = _lib.load()
    cases = [
        ("b200pf_opm_producer", (None, None, None, None, None, None, None, 8, 8, 8, None), "null pointer"),
        ("b200pf_opm_outer", (None, None, None, 8, 8, 8, 8, None), "null or misaligned"),
        ("b200pf_opm_mask_bits", (None, None, 8, 8, None), "bad arguments"),
        ("b200pf_opm_finalize", (None, None, None, None, 8, 0, 8, 8, 1, None), "null or misaligned"),
        ("b200pf_msa_ln_bf16", (None, None, None, None, 8, 8, 8, None), "null or misaligned"),
        ("b200pf_pwa_softmax", (None, None, None, 8, 8, 8, 1e6, None), "bad arguments"),
        ("b200pf_pwa_gate_transpose", (None, None, None, 8, 8, None), "null or misaligned"),
        ("b200pf_msa_swiglu", (None, None, 8, None), "bad arguments"),
        ("b200pf_msa_add_rows", (None, None, 8, 8, 8, None), "bad arguments"),
    ]
    for name, args, text in cases:
        rc = getattr(lib, name)(*args)
        assert rc != 0 and text in _lib.last_error(), (name, rc, _lib.last_error())
    # sizes are checked once the pointers are plausible (16-byte aligned dummies; nothing is dereferenced)
    buf = (ctypes.c_char * 64)()
    p = (ctypes.addressof(buf) + 15) // 16 * 16
    assert lib.b200pf_msa_ln_bf16(p, p, p, p, 4, 9, 12, None) != 0 and "bad sizes" in _lib.last_error()       # np not a multiple of 8
    assert lib.b200pf_pwa_gate_transpose(p, p, p, 4, 12, None) != 0 and "multiple of 8" in _lib.last_error()
    assert lib.b200pf_opm_finalize(p, p, p, p, 1 << 20, 0, 4, 8, 0, None) != 0 and "sequences" in _lib.last_error()
    assert lib.b200pf_opm_outer(p, p, p, 16, 4, 4, 12, None) != 0 and "bad sizes" in _lib.last_error()          # pitch not a multiple of 8
