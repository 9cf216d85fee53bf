"""Host-side weight packing for the b200pf kernels.

Input: the reference's flat state dict for one layer (keys as in tt_bio/reference.py:825-863).
Output: device tensors in the layouts include/b200pf.h documents: bf16 rows grouped the way one
GEMM of a kernel wants them, the 0.5 of sigmoid(x) = 0.5 + 0.5 tanh(x / 2) folded into gate rows,
LayerNorm gains / offsets as fp32 vectors the kernels apply themselves.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

LOG2E = 1.4426950408889634
C_Z = 128
TRI_HEADS, TRI_HEAD_DIM = 4, 32


def pack_trimul(sd: Dict[str, torch.Tensor], pre: str, device) -> Dict[str, torch.Tensor]:
    f = {k: sd[pre + k].detach().float().cpu() for k in
         ("norm_in.weight", "norm_in.bias", "p_in.weight", "g_in.weight", "norm_out.weight", "norm_out.bias",
          "p_out.weight", "g_out.weight")}
    d = f["p_in.weight"].shape[0] // 2
    if d != C_Z or f["p_in.weight"].shape[1] != C_Z:
        raise RuntimeError("the fused triangle-multiplication kernels are built for c_z = hidden = 128")
    # producer: 0.5 * [p_a | g_a | p_b | g_b], 128 rows each, LayerNorm affine applied in the kernel
    w_pg_tc = 0.5 * torch.cat([f["p_in.weight"][:d], f["g_in.weight"][:d], f["p_in.weight"][d:], f["g_in.weight"][d:]], 0)
    # epilogue: raw-x GEMM with 0.5 * W_pout * gamma_out, LayerNorm over channels applied after the GEMM
    w_pout_tc = (0.5 * f["p_out.weight"] * f["norm_out.weight"][None, :]).to(torch.bfloat16)
    wsum_tc = w_pout_tc.float().sum(1)
    wb_tc = 0.5 * (f["p_out.weight"] @ f["norm_out.bias"])
    w_gout_tc = 0.5 * f["g_out.weight"]
    bf = lambda t: t.to(device=device, dtype=torch.bfloat16).contiguous()
    fp = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
    return {"w_pg_tc": bf(w_pg_tc), "w_pout_tc": bf(w_pout_tc), "wsum_tc": fp(wsum_tc), "wb_tc": fp(wb_tc),
            "w_gout_tc": bf(w_gout_tc), "ln_in_gamma": fp(f["norm_in.weight"]), "ln_in_beta": fp(f["norm_in.bias"])}


def pack_triatt(sd: Dict[str, torch.Tensor], pre: str, device) -> Dict[str, torch.Tensor]:
    f = {k: sd[pre + k].detach().float().cpu() for k in
         ("layer_norm.weight", "layer_norm.bias", "linear.weight", "mha.linear_q.weight", "mha.linear_k.weight",
          "mha.linear_v.weight", "mha.linear_g.weight", "mha.linear_o.weight")}
    if f["linear.weight"].shape != (TRI_HEADS, C_Z) or f["mha.linear_q.weight"].shape != (TRI_HEADS * TRI_HEAD_DIM, C_Z):
        raise RuntimeError("the fused triangle-attention kernels are built for c_z = 128 and 4 heads x 32")
    # producer: [q (scaled) | k | 0.5 g | v], LayerNorm affine and the bias heads applied in fp32 in the kernel
    w_tc = torch.cat([f["mha.linear_q.weight"] * (LOG2E / math.sqrt(TRI_HEAD_DIM)), f["mha.linear_k.weight"],
                      0.5 * f["mha.linear_g.weight"], f["mha.linear_v.weight"]], 0)
    return {"w_qkgv_tc": w_tc.to(device=device, dtype=torch.bfloat16).contiguous(),
            "w_bias_f32": (f["linear.weight"] * LOG2E).to(device=device, dtype=torch.float32).contiguous(),
            "ln_gamma": f["layer_norm.weight"].to(device=device, dtype=torch.float32).contiguous(),
            "ln_beta": f["layer_norm.bias"].to(device=device, dtype=torch.float32).contiguous(),
            "w_o": f["mha.linear_o.weight"].to(device=device, dtype=torch.bfloat16).contiguous()}


def pack_transition_z(sd: Dict[str, torch.Tensor], pre: str, device) -> Dict[str, torch.Tensor]:
    f = {k: sd[pre + k].detach().float().cpu() for k in ("norm.weight", "norm.bias", "fc1.weight", "fc2.weight", "fc3.weight")}
    hidden = f["fc1.weight"].shape[0]
    if hidden != 4 * C_Z or f["fc1.weight"].shape[1] != C_Z:
        raise RuntimeError("the fused transition kernel is built for 128 -> 512 -> 128")
    w3 = torch.stack([f["fc3.weight"][:, st * 64:(st + 1) * 64] for st in range(hidden // 64)], 0)   # [8][128][64]
    # per 64-channel chunk [0.5 * fc1 rows | fc2 rows], LayerNorm affine applied in the kernel
    w12_tc = torch.stack([torch.cat([0.5 * f["fc1.weight"][c * 64:(c + 1) * 64], f["fc2.weight"][c * 64:(c + 1) * 64]], 0)
                          for c in range(hidden // 64)], 0)
    return {"w3": w3.to(device=device, dtype=torch.bfloat16).contiguous(),
            "w12_tc": w12_tc.to(device=device, dtype=torch.bfloat16).contiguous(),
            "ln_gamma": f["norm.weight"].to(device=device, dtype=torch.float32).contiguous(),
            "ln_beta": f["norm.bias"].to(device=device, dtype=torch.float32).contiguous()}


def to_device_f32(sd: Dict[str, torch.Tensor], pre: str, device) -> Dict[str, torch.Tensor]:
    """fp32 device copies of every tensor under ``pre`` (keys relative to ``pre``)."""
    return {k[len(pre):]: v.detach().to(device=device, dtype=torch.float32).contiguous()
            for k, v in sd.items() if k.startswith(pre)}
