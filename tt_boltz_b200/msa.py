"""The MSA stack's write into the pair tensor: the outer-product mean, on the b200pf kernels.

``B200OuterProductMean`` keeps the constructor, ``forward(m, mask, chunk_size=None)`` and state-dict keys of the
reference's ``OuterProductMean`` (tt_bio/reference.py:571-669; device form tt_bio/tenstorrent.py:1632-1718) and adds
``add_into(z, m, mask)``, which accumulates straight into a resident fp32 pair tensor the way the MSA layer uses the
result (``z = z + outer_product_mean(m, msa_mask)``, reference.py:1390).

Per call: one producer kernel (LayerNorm, both projections, mask; operands written K-major with the sequence index
contiguous), the mask as bits, and then per block of tokens i the outer products as one GEMM over the sequences
(the triangle-multiplication contraction kernel, each pair's 32 x 32 block contiguous), the projection to 128
channels as a second GEMM of the same kernel, and a finalize kernel (pair counts by popcount, mean, bias, fp32
accumulation).  A block holds up to 1 GB of outer products (2 KB per pair): larger GEMMs ran faster than blocks
small enough to stay in L2 between the two GEMMs (3.5 against 4.0 ms at 1024 tokens x 1024 sequences).
There is no CPU path: tensors must be on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import nn

from ._lib import Planes, call, ptr, stream

C_M, C_HID, C_OUT = 64, 32, 128
OUTER_BLOCK_BYTES = 1 << 30         # outer products of one block of tokens (2 KB per pair)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class B200OuterProductMean(nn.Module):
    """Drop-in for ``OuterProductMean(c_in=64, c_hidden=32, c_out=128)``; other widths are refused."""

    def __init__(self, c_in: int = C_M, c_hidden: int = C_HID, c_out: int = C_OUT, block_tokens: Optional[int] = None) -> None:
        super().__init__()
        if (c_in, c_hidden, c_out) != (C_M, C_HID, C_OUT):
            raise ValueError(f"B200OuterProductMean is built for widths {(C_M, C_HID, C_OUT)}, got {(c_in, c_hidden, c_out)}")
        self.c_hidden = c_hidden
        self.block_tokens = block_tokens
        self.norm = nn.LayerNorm(c_in)
        self.proj_a = nn.Linear(c_in, c_hidden, bias=False)
        self.proj_b = nn.Linear(c_in, c_hidden, bias=False)
        self.proj_o = nn.Linear(c_hidden * c_hidden, c_out)
        self._packed = None

    # -- weights -------------------------------------------------------------------------------------
    def _load_from_state_dict(self, *args, **kwargs):
        self._packed = None
        return super()._load_from_state_dict(*args, **kwargs)

    def _apply(self, fn, *args, **kwargs):
        self._packed = None
        return super()._apply(fn, *args, **kwargs)

    def _pack(self, device):
        if self._packed is None or self._packed["w_ab"].device != device:
            with torch.no_grad():
                f32 = dict(device=device, dtype=torch.float32)
                self._packed = {
                    "gamma": self.norm.weight.detach().to(**f32).contiguous(),
                    "beta": self.norm.bias.detach().to(**f32).contiguous(),
                    "w_ab": torch.cat([self.proj_a.weight, self.proj_b.weight], 0).detach().to(**f32).contiguous(),
                    "w_o": self.proj_o.weight.detach().to(device=device, dtype=torch.bfloat16).contiguous(),
                    "bias": self.proj_o.bias.detach().to(**f32).contiguous(),
                }
        return self._packed

    # -- compute -------------------------------------------------------------------------------------
    def _run(self, z: torch.Tensor, m: torch.Tensor, mask: torch.Tensor, accumulate: bool) -> None:
        """z [N, N, 128] fp32 (written or accumulated into), m [S, N, 64] fp32, mask [S, N]."""
        if not (m.is_cuda and z.is_cuda):
            raise RuntimeError("B200OuterProductMean needs CUDA tensors: the b200pf kernels have no CPU path")
        s_len, n = m.shape[0], m.shape[1]
        if m.shape[2] != C_M or tuple(z.shape) != (n, n, C_OUT) or tuple(mask.shape) != (s_len, n):
            raise ValueError(f"shapes do not fit: m {tuple(m.shape)}, mask {tuple(mask.shape)}, z {tuple(z.shape)}")
        if z.dtype != torch.float32 or not z.is_contiguous():
            raise ValueError("z must be contiguous fp32")
        w = self._pack(m.device)
        m = m.to(torch.float32).contiguous()
        mask_u8 = (mask != 0).to(torch.uint8).contiguous()
        dev, st = m.device, stream()
        pitch = _round_up(s_len, 8)
        a_t = torch.empty(n * C_HID * pitch, dtype=torch.bfloat16, device=dev)
        b_t = torch.empty(n * C_HID * pitch, dtype=torch.bfloat16, device=dev)
        call("b200pf_opm_producer", ptr(m), ptr(mask_u8), ptr(w["gamma"]), ptr(w["beta"]), ptr(w["w_ab"]), ptr(a_t), ptr(b_t),
             s_len, n, pitch, st)
        words = (s_len + 31) // 32
        bits = torch.empty(n * words, dtype=torch.int32, device=dev)
        call("b200pf_opm_mask_bits", ptr(mask_u8), ptr(bits), s_len, n, st)
        k2 = C_HID * C_HID
        blk = self.block_tokens or max(4, OUTER_BLOCK_BYTES // (n * k2 * 2) // 4 * 4)
        blk = min(blk, n)
        x2 = torch.empty(blk * n * k2, dtype=torch.bfloat16, device=dev)
        y = torch.empty(blk * n * C_OUT, dtype=torch.bfloat16, device=dev)
        pw = Planes(ptr(w["w_o"]), C_OUT * k2, 0, k2, C_OUT, k2, 1, 0)
        for i0 in range(0, n, blk):
            ni = min(blk, n - i0)
            call("b200pf_opm_outer", ptr(a_t[i0 * C_HID * pitch:]), ptr(b_t), ptr(x2), s_len, ni, n, pitch, st)
            px = Planes(ptr(x2), ni * n * k2, 0, k2, ni * n, k2, 1, 0)
            call("b200pf_trimul_contract", C.byref(px), C.byref(pw), None, None, ptr(y), ni * n * C_OUT, C_OUT, 0, 0, 1, 0, st)
            call("b200pf_opm_finalize", ptr(y), ptr(bits), ptr(w["bias"]), ptr(z[i0:]), s_len, i0, ni, n, int(accumulate), st)

    def add_into(self, z: torch.Tensor, m: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """z += outer_product_mean(m, mask) in place; z [1, N, N, 128] or [N, N, 128] fp32, m [1, S, N, 64] or [S, N, 64]."""
        zz = z[0] if z.dim() == 4 else z
        mm = m[0] if m.dim() == 4 else m
        mk = mask[0] if mask.dim() == 3 else mask
        with torch.no_grad():
            self._run(zz, mm, mk, accumulate=True)
        return z

    def forward(self, m: torch.Tensor, mask: torch.Tensor, chunk_size: Optional[int] = None) -> torch.Tensor:
        """m [B, S, N, 64], mask [B, S, N] -> [B, N, N, 128] (reference.py:597-669); B must be 1.  ``chunk_size`` only
        bounds the reference's peak memory and is ignored."""
        if m.dim() != 4 or m.shape[0] != 1:
            raise ValueError("B200OuterProductMean.forward takes m of shape [1, S, N, 64]")
        n = m.shape[2]
        out = torch.empty(1, n, n, C_OUT, dtype=torch.float32, device=m.device)
        with torch.no_grad():
            self._run(out[0], m[0], mask[0], accumulate=False)
        return out
