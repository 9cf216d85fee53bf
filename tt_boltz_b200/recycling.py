"""The trunk's recycling loop with the pair tensor resident on the GPU.

The reference runs, per recycle (tt_bio/boltz2.py:5203-5250):

    s = s_init + s_recycle(s_norm(s));   z = z_init + z_recycle(z_norm(z))
    z = z + template_module(z, ...);     z = z + msa_module(z, ...)          (other modules, optional)
    s, z = pairformer_module(s, z, mask=mask, pair_mask=pair_mask)

starting from s = z = 0, ``recycling_steps + 1`` times.  With the Pairformer on the GPU the two recycle
projections are what is left between two trunk passes; running them here too keeps z (512 MiB in fp32 at
N = 1024) on the device from the first recycle to the last instead of crossing PCIe twice per recycle - the same
gain the reference takes from its resident-z loop on its own backend (tt_bio/esmfold2_runtime.py:227-289).
Parameters carry the reference's key names (``s_norm``, ``z_norm``, ``s_recycle``, ``z_recycle``,
``pairformer_module``), so the matching slice of a Boltz-2 checkpoint loads unchanged.

After the last recycle the reference reads the distogram off the resident z (tt_bio/boltz2.py:5250,
``DistogramModule`` :2334-2368): ``B200DistogramModule`` does that on the device too.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
from torch import nn

from . import ops
from ._lib import call, ptr, stream
from .pairformer import B200PairformerModule, _mask_u8


def _ln_linear_residual(x: torch.Tensor, base: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """base + Linear(LayerNorm(x)) in fp32 with the library's kernels; returns a new tensor shaped like base."""
    y = ops.f32_layernorm(x, gamma, beta)
    out = base.clone()
    ops.f32_linear(y, w, out=out.view(-1, out.shape[-1]), accumulate=True)
    return out


class B200RecyclingTrunk(nn.Module):
    """``forward(s_init, z_init, mask, pair_mask, recycling_steps, pair_update=None) -> (s, z)``.

    ``pairformer_module`` is a ``B200PairformerModule`` (one GPU) or a ``ShardedPairformerModule`` (then
    ``z_init`` is THIS rank's row shard [1, N/P, N, C] and so is the returned z).  ``pair_update(z) -> dz`` stands
    for the template and MSA modules of the reference loop, which are not part of this library: it gets the
    resident z as a [1, rows, N, C] fp32 view and returns what is to be added (or None)."""

    def __init__(self, pairformer_module: nn.Module, token_s: int = 384, token_z: int = 128) -> None:
        super().__init__()
        self.token_s, self.token_z = token_s, token_z
        self.s_norm = nn.LayerNorm(token_s)
        self.z_norm = nn.LayerNorm(token_z)
        self.s_recycle = nn.Linear(token_s, token_s, bias=False)
        self.z_recycle = nn.Linear(token_z, token_z, bias=False)
        self.pairformer_module = pairformer_module
        for p in self.parameters():
            p.requires_grad_(False)

    def forward(self, s_init: torch.Tensor, z_init: torch.Tensor, mask: Optional[torch.Tensor] = None,
                pair_mask: Optional[torch.Tensor] = None, recycling_steps: int = 0,
                pair_update: Optional[Callable[[torch.Tensor], Optional[torch.Tensor]]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        if not z_init.is_cuda:
            raise RuntimeError("B200RecyclingTrunk: inputs must be CUDA tensors (there is no CPU path)")
        dev = z_init.device
        pf = self.pairformer_module
        sharded = not isinstance(pf, B200PairformerModule)
        with torch.cuda.device(dev), torch.no_grad():
            f32 = lambda t: t.detach().to(device=dev, dtype=torch.float32).contiguous()
            w = {k: f32(v) for k, v in (("sg", self.s_norm.weight), ("sb", self.s_norm.bias), ("zg", self.z_norm.weight),
                                        ("zb", self.z_norm.bias), ("sw", self.s_recycle.weight), ("zw", self.z_recycle.weight))}
            s0, z0 = f32(s_init[0]), f32(z_init[0])
            s, z = torch.zeros_like(s0), torch.zeros_like(z0)
            for _ in range(recycling_steps + 1):
                s = _ln_linear_residual(s, s0, w["sg"], w["sb"], w["sw"])
                z = _ln_linear_residual(z, z0, w["zg"], w["zb"], w["zw"])
                if pair_update is not None:
                    dz = pair_update(z.unsqueeze(0))
                    if dz is not None:
                        z += dz[0].to(torch.float32)
                if sharded:
                    s, z = pf.forward_sharded(s, z, mask, pair_mask)
                else:
                    pf.run_inplace(s, z, mask, pair_mask)
        return s.unsqueeze(0).to(s_init.dtype), z.unsqueeze(0).to(z_init.dtype)


class B200DistogramModule(nn.Module):
    """``forward(z) -> [1, N, N, num_distograms, num_bins]``: ``Linear(z + z^T)`` with the reference's parameter names
    (``distogram.weight``, ``distogram.bias``; tt_bio/boltz2.py:2334-2368), in fp32 on the library's kernels: the
    symmetrisation is one transpose-accumulate pass over a copy of z, the projection one 3xTF32 GEMM with its bias."""

    def __init__(self, token_z: int = 128, num_bins: int = 64, num_distograms: int = 1) -> None:
        super().__init__()
        self.token_z, self.num_bins, self.num_distograms = token_z, num_bins, num_distograms
        self.distogram = nn.Linear(token_z, num_distograms * num_bins)
        for p in self.parameters():
            p.requires_grad_(False)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        if not z.is_cuda:
            raise RuntimeError("B200DistogramModule: inputs must be CUDA tensors (there is no CPU path)")
        if z.dim() != 4 or z.shape[0] != 1 or z.shape[1] != z.shape[2] or z.shape[3] != self.token_z:
            raise ValueError(f"B200DistogramModule: z must be [1, N, N, {self.token_z}], got {tuple(z.shape)}")
        dev, n = z.device, z.shape[1]
        with torch.cuda.device(dev), torch.no_grad():
            f32 = lambda t: t.detach().to(device=dev, dtype=torch.float32).contiguous()
            z0 = f32(z[0])
            sym = z0.clone()
            call("b200pf_f32_transpose01", ptr(z0), ptr(sym), n, self.token_z, 1, stream())      # sym += z^T
            out = ops.f32_linear(sym, f32(self.distogram.weight), f32(self.distogram.bias))
        return out.view(1, n, n, self.num_distograms, self.num_bins).to(z.dtype)
