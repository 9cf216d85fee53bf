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


# ------------------------------------------------------------------------------------------------
# The MSA layer: pair-weighted averaging and transition on m, outer-product mean and a pair block on z
# ------------------------------------------------------------------------------------------------
ROWS_PER_CHUNK = 1 << 20           # (sequence, token) rows whose bf16 intermediates are held at a time


def _gemm(a, a_rows, k, b, b_rows, x, channels=1, a_plane=None, b_plane=None, a_pitch=None, b_pitch=None,
          x_plane=None, x_pitch=None, cols=None) -> None:
    """x[d][i][j] = sum_k a[d][i][k] b[d][j][k] through the contraction kernel (bf16 operands, fp32 accumulation)."""
    a_pitch, b_pitch = a_pitch or k, b_pitch or k
    pa = Planes(ptr(a), a_plane if a_plane is not None else a_rows * a_pitch, 0, a_pitch, a_rows, cols or k, 1, 0)
    pb = Planes(ptr(b), b_plane if b_plane is not None else b_rows * b_pitch, 0, b_pitch, b_rows, cols or k, 1, 0)
    x_pitch = x_pitch or b_rows
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x),
         x_plane if x_plane is not None else a_rows * x_pitch, x_pitch, 0, 0, channels, 0, stream())


def _check_m(m: torch.Tensor) -> None:
    if not m.is_cuda:
        raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
    if m.dim() != 3 or m.shape[2] != C_M or m.dtype != torch.float32 or not m.is_contiguous():
        raise ValueError("m must be a contiguous fp32 tensor [S, N, 64]")


class B200PairWeightedAveraging(nn.Module):
    """Drop-in for ``PairWeightedAveraging(c_m=64, c_z=128, c_h=32, num_heads=8)`` (tt_bio/reference.py:672-800; device
    form tt_bio/tenstorrent.py:1542-1629): ``forward(m, z, mask, chunk_heads)`` returns the update of m, ``add_into``
    accumulates it into a resident fp32 m."""

    def __init__(self, c_m: int = C_M, c_z: int = 128, c_h: int = 32, num_heads: int = 8, inf: float = 1e6) -> None:
        super().__init__()
        if (c_m, c_z, c_h, num_heads) != (C_M, 128, 32, 8):
            raise ValueError(f"B200PairWeightedAveraging is built for (c_m, c_z, c_h, heads) = (64, 128, 32, 8), got {(c_m, c_z, c_h, num_heads)}")
        self.c_m, self.c_z, self.c_h, self.num_heads, self.inf = c_m, c_z, c_h, num_heads, inf
        self.norm_m = nn.LayerNorm(c_m)
        self.norm_z = nn.LayerNorm(c_z)
        self.proj_m = nn.Linear(c_m, c_h * num_heads, bias=False)
        self.proj_g = nn.Linear(c_m, c_h * num_heads, bias=False)
        self.proj_z = nn.Linear(c_z, num_heads, bias=False)
        self.proj_o = nn.Linear(c_h * num_heads, c_m, bias=False)
        self._packed = None

    def _load_from_state_dict(self, *args, **kwargs):
        self._packed = None
        return super()._load_from_state_dict(*args, **kwargs)

    def _apply(self, fn, *args, **kwargs):
        self._packed = None
        return super()._apply(fn, *args, **kwargs)

    def _pack(self, device):
        if self._packed is None or self._packed["w_mg"].device != device:
            with torch.no_grad():
                f32 = dict(device=device, dtype=torch.float32)
                self._packed = {
                    "gm": self.norm_m.weight.detach().to(**f32).contiguous(), "bm": self.norm_m.bias.detach().to(**f32).contiguous(),
                    "gz": self.norm_z.weight.detach().to(**f32).contiguous(), "bz": self.norm_z.bias.detach().to(**f32).contiguous(),
                    "w_mg": torch.cat([self.proj_m.weight, self.proj_g.weight], 0).detach().to(device=device, dtype=torch.bfloat16).contiguous(),
                    # the LayerNorm + head projection kernel is built for 16 heads: 8 real rows, 8 zero rows
                    "w_z": torch.cat([self.proj_z.weight.detach().to(**f32), torch.zeros(8, self.c_z, **f32)], 0).contiguous(),
                    "w_o": self.proj_o.weight.detach().to(device=device, dtype=torch.bfloat16).contiguous(),
                }
        return self._packed

    def _run(self, m: torch.Tensor, z: torch.Tensor, mask_u8: torch.Tensor) -> None:
        """m [S, N, 64] fp32 updated in place from z [N, N, 128] fp32 and the pair mask [N, N] (uint8)."""
        _check_m(m)
        s_len, n = m.shape[0], m.shape[1]
        if tuple(z.shape) != (n, n, 128) or z.dtype != torch.float32 or not z.is_contiguous():
            raise ValueError("z must be a contiguous fp32 tensor [N, N, 128]")
        w = self._pack(m.device)
        dev, st, heads = m.device, stream(), self.num_heads
        np_, pw = _round_up(n, 32), _round_up(n, 8)          # the projected rows are written in column groups of np
        logits = torch.empty(16 * n * n, dtype=torch.float32, device=dev)
        call("b200pf_ln_proj_heads", ptr(z), ptr(w["gz"]), ptr(w["bz"]), ptr(w["w_z"]), ptr(logits), n * n, n * n, 128, 16, st)
        wt = torch.empty(heads * n * pw, dtype=torch.bfloat16, device=dev)
        call("b200pf_pwa_softmax", ptr(logits), ptr(mask_u8), ptr(wt), n, pw, heads, float(self.inf), st)
        sc = max(1, min(s_len, ROWS_PER_CHUNK // np_))
        ln = torch.empty(sc * np_ * C_M, dtype=torch.bfloat16, device=dev)
        vg = torch.empty(512 * sc * np_, dtype=torch.bfloat16, device=dev)
        o = torch.empty(256 * sc * np_, dtype=torch.bfloat16, device=dev)
        val = torch.empty(sc * np_ * 256, dtype=torch.bfloat16, device=dev)
        t = torch.empty(sc * np_ * C_M, dtype=torch.bfloat16, device=dev)
        for s0 in range(0, s_len, sc):
            ns = min(sc, s_len - s0)
            p = ns * np_
            call("b200pf_msa_ln_bf16", ptr(m[s0:]), ptr(w["gm"]), ptr(w["bm"]), ptr(ln), ns, n, np_, st)
            # [v heads 0-7 ; g heads 0-7][s][d][token]: rows (head, d) in groups of 32, columns (s, token) in groups of np
            pa = Planes(ptr(w["w_mg"]), 512 * C_M, 0, C_M, 512, C_M, 1, 0)
            pb = Planes(ptr(ln), p * C_M, 0, C_M, p, C_M, 1, 0)
            call("b200pf_gemm_grouped", C.byref(pa), C.byref(pb), ptr(vg), 0, np_, 32, ns * 32 * np_, np_, 32 * np_, 1, st)
            _gemm(vg, self.c_h * ns, n, wt, n, o, channels=heads, a_plane=self.c_h * p, a_pitch=np_,
                  b_plane=n * pw, b_pitch=pw, x_plane=self.c_h * p, x_pitch=np_, cols=n)
            call("b200pf_pwa_gate_transpose", ptr(o), ptr(vg[256 * p:]), ptr(val), ns, np_, st)        # sigmoid(g) * o, K-major
            _gemm(val, p, 256, w["w_o"], C_M, t)
            call("b200pf_msa_add_rows", ptr(m[s0:]), ptr(t), ns, n, np_, st)

    def add_into(self, m: torch.Tensor, z: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """m += pair_weighted_averaging(m, z, mask) in place; m [S, N, 64] fp32, z [N, N, 128] fp32, mask [N, N]."""
        with torch.no_grad():
            self._run(m, z, (mask != 0).to(torch.uint8).contiguous())
        return m

    def forward(self, m: torch.Tensor, z: torch.Tensor, mask: torch.Tensor, chunk_heads: bool = False) -> torch.Tensor:
        """m [1, S, N, 64], z [1, N, N, 128], mask [1, N, N] -> the update [1, S, N, 64] (reference.py:727-800)."""
        if m.dim() != 4 or m.shape[0] != 1:
            raise ValueError("B200PairWeightedAveraging.forward takes m of shape [1, S, N, 64]")
        if not m.is_cuda:
            raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
        with torch.no_grad():
            m0 = m[0].to(torch.float32).contiguous()
            work = m0.clone()
            self._run(work, z[0].to(torch.float32).contiguous(), (mask[0] != 0).to(torch.uint8).contiguous())
            return (work - m0)[None]


class B200MSATransition(nn.Module):
    """Drop-in for ``Transition(dim=64, hidden=256)`` on the MSA activations (tt_bio/boltz2.py:1188-1258):
    ``forward(x, chunk_size)`` returns the update, ``add_into`` accumulates it into a resident fp32 m."""

    def __init__(self, dim: int = C_M, hidden: int = 256, out_dim: Optional[int] = None) -> None:
        super().__init__()
        if (dim, hidden, out_dim or dim) != (C_M, 256, C_M):
            raise ValueError(f"B200MSATransition is built for (dim, hidden) = (64, 256), got {(dim, hidden, out_dim)}")
        self.norm = nn.LayerNorm(dim, eps=1e-5)
        self.fc1 = nn.Linear(dim, hidden, bias=False)
        self.fc2 = nn.Linear(dim, hidden, bias=False)
        self.fc3 = nn.Linear(hidden, dim, bias=False)
        self.hidden = hidden
        self._packed = None

    def _load_from_state_dict(self, *args, **kwargs):
        self._packed = None
        return super()._load_from_state_dict(*args, **kwargs)

    def _apply(self, fn, *args, **kwargs):
        self._packed = None
        return super()._apply(fn, *args, **kwargs)

    def _pack(self, device):
        if self._packed is None or self._packed["w12"].device != device:
            with torch.no_grad():
                bf = dict(device=device, dtype=torch.bfloat16)
                self._packed = {
                    "g": self.norm.weight.detach().to(device=device, dtype=torch.float32).contiguous(),
                    "b": self.norm.bias.detach().to(device=device, dtype=torch.float32).contiguous(),
                    "w12": torch.cat([self.fc1.weight, self.fc2.weight], 0).detach().to(**bf).contiguous(),
                    "w3": self.fc3.weight.detach().to(**bf).contiguous(),
                }
        return self._packed

    def _run(self, m: torch.Tensor) -> None:
        _check_m(m)
        s_len, n = m.shape[0], m.shape[1]
        w = self._pack(m.device)
        dev, st = m.device, stream()
        np_ = _round_up(n, 8)
        sc = max(1, min(s_len, ROWS_PER_CHUNK // np_))
        ln = torch.empty(sc * np_ * C_M, dtype=torch.bfloat16, device=dev)
        h12 = torch.empty(sc * np_ * 512, dtype=torch.bfloat16, device=dev)
        hsw = torch.empty(sc * np_ * 256, dtype=torch.bfloat16, device=dev)
        t = torch.empty(sc * np_ * C_M, dtype=torch.bfloat16, device=dev)
        for s0 in range(0, s_len, sc):
            ns = min(sc, s_len - s0)
            p = ns * np_
            call("b200pf_msa_ln_bf16", ptr(m[s0:]), ptr(w["g"]), ptr(w["b"]), ptr(ln), ns, n, np_, st)
            _gemm(ln, p, C_M, w["w12"], 512, h12)
            call("b200pf_msa_swiglu", ptr(h12), ptr(hsw), p, st)
            _gemm(hsw, p, 256, w["w3"], C_M, t)
            call("b200pf_msa_add_rows", ptr(m[s0:]), ptr(t), ns, n, np_, st)

    def add_into(self, m: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            self._run(m)
        return m

    def forward(self, x: torch.Tensor, chunk_size: Optional[int] = None) -> torch.Tensor:
        """x [1, S, N, 64] -> the update [1, S, N, 64]; ``chunk_size`` only bounds the reference's memory."""
        if x.dim() != 4 or x.shape[0] != 1:
            raise ValueError("B200MSATransition.forward takes x of shape [1, S, N, 64]")
        if not x.is_cuda:
            raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
        with torch.no_grad():
            x0 = x[0].to(torch.float32).contiguous()
            work = x0.clone()
            self._run(work)
            return (work - x0)[None]


class B200MSALayer(nn.Module):
    """One block of the MSA module with the reference's constructor, sub-module names and
    ``forward(z, m, token_mask, msa_mask, ...) -> (z, m)`` (tt_bio/reference.py:1311-1397; device form
    tt_bio/tenstorrent.py:1721-1790): pair-weighted averaging and transition on m, then the outer-product mean and a
    pair-only Pairformer block on z.  Inference only: the dropout masks of the reference are the identity in eval mode."""

    def __init__(self, msa_s: int = C_M, token_z: int = 128, msa_dropout: float = 0.0, z_dropout: float = 0.0,
                 pairwise_head_width: int = 32, pairwise_num_heads: int = 4, precision: str = "bf16") -> None:
        super().__init__()
        from .pairformer import B200PairformerNoSeqLayer
        self.msa_dropout = msa_dropout
        self.msa_transition = B200MSATransition(dim=msa_s, hidden=msa_s * 4)
        self.pair_weighted_averaging = B200PairWeightedAveraging(c_m=msa_s, c_z=token_z, c_h=32, num_heads=8)
        self.pairformer_layer = B200PairformerNoSeqLayer(token_z, z_dropout, pairwise_head_width, pairwise_num_heads,
                                                         precision=precision)
        self.outer_product_mean = B200OuterProductMean(c_in=msa_s, c_hidden=32, c_out=token_z)

    def forward_inplace(self, z: torch.Tensor, m: torch.Tensor, token_mask: torch.Tensor, msa_mask: torch.Tensor) -> None:
        """z [N, N, 128] and m [S, N, 64], contiguous fp32, updated where they are; token_mask [N, N], msa_mask [S, N]."""
        from .pairformer import _run_layers
        self.pair_weighted_averaging.add_into(m, z, token_mask)
        self.msa_transition.add_into(m)
        self.outer_product_mean.add_into(z, m, msa_mask)
        _run_layers([self.pairformer_layer], None, z, None, token_mask[None], inplace=True)

    def forward(self, z: torch.Tensor, m: torch.Tensor, token_mask: torch.Tensor, msa_mask: torch.Tensor,
                chunk_heads_pwa: bool = False, chunk_size_transition_z: Optional[int] = None,
                chunk_size_transition_msa: Optional[int] = None, chunk_size_outer_product: Optional[int] = None,
                chunk_size_tri_attn: Optional[int] = None, use_kernels: bool = False):
        """z [1, N, N, 128], m [1, S, N, 64], token_mask [1, N, N], msa_mask [1, S, N] -> (z, m); the chunk sizes only
        bound the reference's memory and are ignored."""
        if not (z.is_cuda and m.is_cuda):
            raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
        with torch.no_grad():
            zw = z[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            mw = m[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            self.forward_inplace(zw, mw, token_mask[0], msa_mask[0])
        return zw[None], mw[None]


class B200MSAStack(nn.Module):
    """The ``layers`` of the reference's MSA module (tt_bio/reference.py:1187-1201, loop at :1279-1307) on resident
    tensors: ``forward(z, m, token_mask, msa_mask) -> z`` runs every block on copies, ``run_inplace`` on the caller's
    fp32 z [N, N, 128] and m [S, N, 64], for callers that keep the embedded MSA on the GPU across recycles
    (``B200MSAModule`` embeds the features and runs the same blocks)."""

    def __init__(self, msa_blocks: int = 4, msa_s: int = C_M, token_z: int = 128, msa_dropout: float = 0.0, z_dropout: float = 0.0,
                 pairwise_head_width: int = 32, pairwise_num_heads: int = 4, precision: str = "bf16") -> None:
        super().__init__()
        self.msa_blocks = msa_blocks
        self.layers = nn.ModuleList(B200MSALayer(msa_s, token_z, msa_dropout, z_dropout, pairwise_head_width,
                                                 pairwise_num_heads, precision) for _ in range(msa_blocks))

    def run_inplace(self, z: torch.Tensor, m: torch.Tensor, token_mask: torch.Tensor, msa_mask: torch.Tensor) -> None:
        for layer in self.layers:
            layer.forward_inplace(z, m, token_mask, msa_mask)

    def forward(self, z: torch.Tensor, m: torch.Tensor, token_mask: torch.Tensor, msa_mask: torch.Tensor) -> torch.Tensor:
        """z [1, N, N, 128], m [1, S, N, 64], token_mask [1, N, N], msa_mask [1, S, N] -> z (what MSAModule.forward returns)."""
        if not (z.is_cuda and m.is_cuda):
            raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
        with torch.no_grad():
            zw = z[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            mw = m[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            self.run_inplace(zw, mw, token_mask[0], msa_mask[0])
        return zw[None]


NUM_TOKENS = 33                    # residue / nucleotide / gap classes of the MSA one-hot (tt_bio/data/const.py:157)


class B200MSAModule(nn.Module):
    """Drop-in for the reference's ``MSAModule`` (tt_bio/reference.py:1150-1308; device form
    tt_bio/tenstorrent.py:2524-2621): the MSA features are embedded (``msa_proj`` of the one-hot residues, deletion and
    pairing features, plus ``s_proj`` of the single representation for every sequence) and ``msa_blocks`` MSA layers
    run on resident tensors; ``forward(z, emb, feats, use_kernels=False)`` returns the pair tensor after the last
    block, which the trunk adds to z (tt_bio/boltz2.py:5230).  The one-hot and the concatenation of the raw features
    are torch indexing at the boundary; both projections and everything after run on the b200pf kernels."""

    def __init__(self, msa_s: int = C_M, token_z: int = 128, token_s: int = 384, msa_blocks: int = 4, msa_dropout: float = 0.0,
                 z_dropout: float = 0.0, pairwise_head_width: int = 32, pairwise_num_heads: int = 4,
                 activation_checkpointing: bool = False, use_paired_feature: bool = True, subsample_msa: bool = False,
                 num_subsampled_msa: int = 1024, precision: str = "bf16", **kwargs) -> None:
        super().__init__()
        self.msa_blocks, self.use_paired_feature = msa_blocks, use_paired_feature
        self.subsample_msa, self.num_subsampled_msa = subsample_msa, num_subsampled_msa
        self.s_proj = nn.Linear(token_s, msa_s, bias=False)
        self.msa_proj = nn.Linear(NUM_TOKENS + 2 + int(use_paired_feature), msa_s, bias=False)
        self.layers = nn.ModuleList(B200MSALayer(msa_s, token_z, msa_dropout, z_dropout, pairwise_head_width,
                                                 pairwise_num_heads, precision) for _ in range(msa_blocks))

    def embed(self, emb: torch.Tensor, feats) -> torch.Tensor:
        """m [S, N, 64] fp32 from the single representation emb [1, N, token_s] and the MSA features (reference.py:1252-1276)."""
        from . import ops
        msa = torch.nn.functional.one_hot(feats["msa"][0], num_classes=NUM_TOKENS).to(torch.float32)
        parts = [msa, feats["has_deletion"][0].unsqueeze(-1).float(), feats["deletion_value"][0].unsqueeze(-1).float()]
        if self.use_paired_feature:
            parts.append(feats["msa_paired"][0].unsqueeze(-1).float())
        raw = torch.cat(parts, dim=-1)                                      # [S, N, 35 or 36]
        if raw.shape[-1] % 4:                                               # the linear kernel wants 16-byte rows
            raw = torch.nn.functional.pad(raw, (0, 4 - raw.shape[-1] % 4))
        w = self.msa_proj.weight.detach().to(device=raw.device, dtype=torch.float32)
        if w.shape[1] != raw.shape[-1]:
            w = torch.nn.functional.pad(w, (0, raw.shape[-1] - w.shape[1]))
        s_len, n = raw.shape[0], raw.shape[1]
        m = ops.f32_linear(raw.contiguous(), w.contiguous()).view(s_len, n, C_M)
        e = ops.f32_linear(emb[0].to(torch.float32).contiguous(),
                           self.s_proj.weight.detach().to(device=raw.device, dtype=torch.float32).contiguous())
        call("b200pf_msa_add_token_rows", ptr(m), ptr(e), s_len, n, stream())
        return m

    def forward(self, z: torch.Tensor, emb: torch.Tensor, feats, use_kernels: bool = False) -> torch.Tensor:
        """z [1, N, N, 128], emb [1, N, token_s], feats with ``msa`` [1, S, N] (int64), ``has_deletion``,
        ``deletion_value``, ``msa_paired``, ``msa_mask`` [1, S, N] and ``token_pad_mask`` [1, N] -> z [1, N, N, 128]."""
        if not (z.is_cuda and emb.is_cuda and feats["msa"].is_cuda):
            raise RuntimeError("the MSA kernels need CUDA tensors: the b200pf kernels have no CPU path")
        with torch.no_grad():
            msa_mask = feats["msa_mask"][0]
            if self.subsample_msa:                                          # reference.py:1269-1272
                idx = torch.randperm(feats["msa"].shape[1], device=z.device)[: self.num_subsampled_msa]
                feats = {k: (v[:, idx] if k in ("msa", "has_deletion", "deletion_value", "msa_paired") else v) for k, v in feats.items()}
                msa_mask = msa_mask[idx]
            tok = feats["token_pad_mask"][0].float()
            token_mask = tok[:, None] * tok[None, :]
            m = self.embed(emb, feats)
            zw = z[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            for layer in self.layers:
                layer.forward_inplace(zw, m, token_mask, msa_mask)
        return zw[None]
