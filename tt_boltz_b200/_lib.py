"""ctypes binding of libb200pf.so (the C ABI declared in include/b200pf.h).

There is no fallback: if the shared library is missing and cannot be built, importing the
binding raises.  Every call checks the status code and raises ``RuntimeError`` with the
library's own message.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200pf.so")

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class Planes(C.Structure):
    """Mirror of ``b200pf_planes``."""
    _fields_ = [("ptr", _vp), ("plane_stride", _ll), ("seg_stride", _ll), ("pitch", _i), ("rows", _i),
                ("cols", _i), ("nseg", _i), ("seg_is_k", _i)]


class PeerSync(C.Structure):
    """Mirror of ``b200pf_peer_sync``."""
    _fields_ = [("pad_ptrs", C.POINTER(C.c_ulonglong)), ("generation", C.c_uint), ("timeout_ns", _ll), ("channel", _i)]


class PlaneOut(C.Structure):
    """Mirror of ``b200pf_plane_out``."""
    _fields_ = [("ptr", _vp), ("plane_stride", _ll), ("group_stride", _ll), ("row_group", _i)]


# name -> argtypes (all return int unless listed in _RESTYPES)
SIGNATURES = {
    "b200pf_version": [],
    "b200pf_last_error": [],
    "b200pf_launch_count": [],
    "b200pf_device_status": [_vp],
    "b200pf_f32_layernorm": [_vp, _vp, _vp, _vp, _ll, _i, _vp],
    "b200pf_f32_linear": [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp],
    "b200pf_f32_gate": [_vp, _vp, _vp, _vp, _ll, _i, _i, _vp],
    "b200pf_f32_trimul_contract": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "b200pf_f32_attention": [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _i, _i, _i, _i, _i,
                             _ll, _ll, _f, _f, _i, _vp],
    "b200pf_f32_transpose01": [_vp, _vp, _i, _i, _i, _vp],
    "b200pf_f32_linear_t": [_vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _vp],
    "b200pf_f32_gate_strided": [_vp, _ll, _vp, _ll, _vp, _ll, _ll, _i, _i, _vp],
    "b200pf_f32_sattention": [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _ll, _vp, _i, _i, _i, _i, _f, _f, _vp],
    "b200pf_ln_proj_heads": [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _vp],
    "b200pf_trimul_producer": [_vp, _vp, _vp, _vp, _vp, C.POINTER(PlaneOut), C.POINTER(PlaneOut), _i, _i, _i, _i, _vp],
    "b200pf_trimul_contract": [C.POINTER(Planes), C.POINTER(Planes), _vp, _vp, _vp, _ll, _i, _i, _ll, _i, _i, _vp],
    "b200pf_mx_scale_bytes": [_i, _i, _i],
    "b200pf_msa_ln_bf16": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "b200pf_pwa_softmax": [_vp, _vp, _vp, _i, _i, _i, C.c_float, _vp],
    "b200pf_pwa_gate_transpose": [_vp, _vp, _vp, _i, _i, _vp],
    "b200pf_gemm_grouped": [C.POINTER(Planes), C.POINTER(Planes), _vp, _ll, _i, _i, _ll, _i, _ll, _i, _vp],
    "b200pf_msa_swiglu": [_vp, _vp, _ll, _vp],
    "b200pf_msa_add_rows": [_vp, _vp, _i, _i, _i, _vp],
    "b200pf_msa_add_token_rows": [_vp, _vp, _i, _i, _vp],
    "b200pf_opm_producer": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "b200pf_opm_outer": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "b200pf_opm_mask_bits": [_vp, _vp, _i, _i, _vp],
    "b200pf_opm_finalize": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "b200pf_trimul_producer_mx": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp],
    "b200pf_mx_dequant": [_vp, _vp, _vp, _ll, _i, _ll, _i, _i, _i, _i, _vp],
    "b200pf_trimul_epilogue_tc": [_vp, _vp, _ll, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "b200pf_triatt_producer": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _vp],
    "b200pf_triatt_producer_bf16z": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _vp],
    "b200pf_triatt_core_tc4": [_vp, _vp, _vp, _i, _vp, _ll, _ll, _vp, _i, _vp, _ll, _ll, _i, _i, _vp],
    "b200pf_triatt_epilogue": [_vp, _vp, _vp, _vp, _ll, _vp],
    "b200pf_triatt_epilogue_update": [_vp, _vp, _vp, _vp, _ll, _vp],
    "b200pf_add_bf16": [_vp, _vp, _ll, _vp],
    "b200pf_peer_scatter_strided_f32_bf16_sync": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _ll, _ll, _ll, _ll, _i, _i, C.POINTER(PeerSync), _vp],
    "b200pf_transition_z_tc": [_vp, _vp, _vp, _vp, _vp, _ll, _vp],
    "b200pf_peer_scatter": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _i, _vp],
    "b200pf_peer_broadcast": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _i, _vp],
    "b200pf_peer_scatter_strided": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _ll, _ll, _ll, _ll, _i, _i, _vp],
    "b200pf_peer_barrier": [C.POINTER(C.c_ulonglong), C.c_uint, _i, _i, _ll, _vp],
    "b200pf_peer_scatter_sync": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _i, C.POINTER(PeerSync), _vp],
    "b200pf_peer_broadcast_sync": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _i, C.POINTER(PeerSync), _vp],
    "b200pf_peer_scatter_strided_sync": [_vp, C.POINTER(C.c_ulonglong), _ll, _i, _ll, _ll, _ll, _ll, _i, _i, C.POINTER(PeerSync), _vp],
    "b200pf_tri_mul_noalloc": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
}
_RESTYPES = {"b200pf_last_error": C.c_char_p, "b200pf_launch_count": _ll, "b200pf_mx_scale_bytes": _ll}

_lib: Optional[C.CDLL] = None


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first if needed) the shared library and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if build_if_missing:
        # build() is a no-op when the stamp over the sources matches, so a library left over from before a
        # source edit is never loaded silently; without nvcc an existing library is used as it is
        from . import build as _build
        if _build.have_nvcc() or not os.path.exists(LIB_PATH):
            _build.build()
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing; run `python -m tt_boltz_b200.build`")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = the .so does not export the symbol
        fn.argtypes = args
        fn.restype = _RESTYPES.get(name, _i)
    _lib = lib
    return lib


def last_error() -> str:
    return load().b200pf_last_error().decode(errors="replace")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device address of a contiguous CUDA tensor (None -> NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("b200pf kernels take CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError("b200pf kernels take contiguous tensors")
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class KernelTimer:
    """Optional per-entry-point timing with CUDA events on the launching stream (benchmarks)."""

    def __init__(self) -> None:
        self.events = []          # (name, start, end)

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.events:
            ms, cnt = out.get(name, (0.0, 0))
            out[name] = (ms + a.elapsed_time(b), cnt + 1)
        return out


timer: Optional[KernelTimer] = None


def call(name: str, *args) -> None:
    t = timer
    if t is not None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with status {rc}: {last_error()}")
    if t is not None:
        b.record()
        t.events.append((name, a, b))


def launch_count() -> int:
    return int(load().b200pf_launch_count())


def device_status() -> int:
    """Synchronise the current stream and return the device status word (0 = clean)."""
    return int(load().b200pf_device_status(stream()))
