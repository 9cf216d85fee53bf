"""Checkpoint key remaps of the sibling models whose trunks are built from the same pair operations.

The reference runs Protenix-v2 (c_z = 256, 8 triangle-attention heads, 48 blocks) and the ESMFold2 folding trunk
(triangle multiplications + SwiGLU transition only, c_z = 256) on its Pairformer primitives after renaming their
checkpoint keys (tt_bio/protenix_weights.py:17-137, tt_bio/esmfold2.py:102-126).  The same renames are expressed
here as tables, so that such a checkpoint loads into ``B200PairformerModule`` / ``B200PairUpdateBlock`` /
``B200OuterProductMean`` / ``B200PairWeightedAveraging`` with ``load_state_dict(strict=True)``.  These widths run on
the un-fused fp32 kernels (``precision="fp32"`` or ``"auto"``).

A table maps OUR key to the source key, or to a tuple of source keys whose rows are concatenated in that order.
"""
from __future__ import annotations

from typing import Dict, Mapping, Tuple, Union

import torch

Source = Union[str, Tuple[str, ...]]

# OpenFold-style triangle multiplication: separate a / b projections -> [a-side ; b-side] rows
TRIANGLE_MULTIPLICATION: Dict[str, Source] = {
    "norm_in.weight": "layer_norm_in.weight", "norm_in.bias": "layer_norm_in.bias",
    "norm_out.weight": "layer_norm_out.weight", "norm_out.bias": "layer_norm_out.bias",
    "p_in.weight": ("linear_a_p.weight", "linear_b_p.weight"),
    "g_in.weight": ("linear_a_g.weight", "linear_b_g.weight"),
    "p_out.weight": "linear_z.weight", "g_out.weight": "linear_g.weight",
}
TRANSITION: Dict[str, Source] = {
    "norm.weight": "layernorm1.weight", "norm.bias": "layernorm1.bias",
    "fc1.weight": "linear_no_bias_a.weight", "fc2.weight": "linear_no_bias_b.weight", "fc3.weight": "linear_no_bias.weight",
}
ATTENTION_PAIR_BIAS: Dict[str, Source] = {
    "proj_q.weight": "attention.linear_q.weight", "proj_q.bias": "attention.linear_q.bias",
    "proj_k.weight": "attention.linear_k.weight", "proj_v.weight": "attention.linear_v.weight",
    "proj_g.weight": "attention.linear_g.weight", "proj_o.weight": "attention.linear_o.weight",
    "proj_z.0.weight": "layernorm_z.weight", "proj_z.0.bias": "layernorm_z.bias",
    "proj_z.1.weight": "linear_nobias_z.weight",
}
OUTER_PRODUCT_MEAN: Dict[str, Source] = {
    "norm.weight": "layer_norm.weight", "norm.bias": "layer_norm.bias",
    "proj_a.weight": "linear_1.weight", "proj_b.weight": "linear_2.weight",
    "proj_o.weight": "linear_out.weight", "proj_o.bias": "linear_out.bias",
}
PAIR_WEIGHTED_AVERAGING: Dict[str, Source] = {
    "norm_m.weight": "layernorm_m.weight", "norm_m.bias": "layernorm_m.bias",
    "norm_z.weight": "layernorm_z.weight", "norm_z.bias": "layernorm_z.bias",
    "proj_m.weight": "linear_no_bias_mv.weight", "proj_g.weight": "linear_no_bias_mg.weight",
    "proj_z.weight": "linear_no_bias_z.weight", "proj_o.weight": "linear_no_bias_out.weight",
}


def _sub(sd: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    p = prefix + "."
    return {k[len(p):]: v for k, v in sd.items() if k.startswith(p)}


def apply_table(sd: Mapping[str, torch.Tensor], table: Mapping[str, Source], defaults: Mapping[str, str] = ()) -> Dict[str, torch.Tensor]:
    """Rename / concatenate according to a table.  ``defaults`` names OUR keys that may be absent in the source and
    are then zeros shaped like another of OUR keys (a LayerNorm without an offset)."""
    out: Dict[str, torch.Tensor] = {}
    for ours, src in table.items():
        if isinstance(src, tuple):
            out[ours] = torch.cat([sd[s] for s in src], dim=0)
        elif src in sd:
            out[ours] = sd[src]
        elif ours in dict(defaults):
            continue
        else:
            raise KeyError(f"source checkpoint has no '{src}' (wanted for '{ours}')")
    for ours, like in dict(defaults).items():
        if ours not in out:
            out[ours] = torch.zeros_like(out[like])
    return out


def protenix_pair_stack(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A pair-only Protenix block (MSA pair stack, template stack) -> keys of ``B200PairformerNoSeqLayer``
    (tt_bio/protenix_weights.py:120-137).  The triangle-attention keys are the same in both."""
    out: Dict[str, torch.Tensor] = {}
    for name in ("tri_mul_out", "tri_mul_in"):
        out.update({f"{name}.{k}": v for k, v in apply_table(_sub(sd, name), TRIANGLE_MULTIPLICATION).items()})
    for name in ("tri_att_start", "tri_att_end"):
        out.update({f"{name}.{k}": v for k, v in _sub(sd, name).items()})
    out.update({f"transition_z.{k}": v for k, v in apply_table(_sub(sd, "pair_transition"), TRANSITION).items()})
    return out


def protenix_pairformer_block(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A Protenix PairformerBlock with its single track -> keys of ``B200PairformerLayer``
    (tt_bio/protenix_weights.py:70-93)."""
    out = protenix_pair_stack(sd)
    apb = _sub(sd, "attention_pair_bias")
    out["pre_norm_s.weight"], out["pre_norm_s.bias"] = apb["layernorm_a.weight"], apb["layernorm_a.bias"]
    out.update({f"attention.{k}": v for k, v in
                apply_table(apb, ATTENTION_PAIR_BIAS, defaults={"proj_z.0.bias": "proj_z.0.weight"}).items()})
    out.update({f"transition_s.{k}": v for k, v in apply_table(_sub(sd, "single_transition"), TRANSITION).items()})
    return out


def protenix_outer_product_mean(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return apply_table(sd, OUTER_PRODUCT_MEAN)


def protenix_pair_weighted_averaging(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return apply_table(sd, PAIR_WEIGHTED_AVERAGING)


def esmfold2_pair_update_block(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """One block of the ESMFold2 folding trunk -> keys of ``B200PairUpdateBlock`` (tt_bio/esmfold2.py:102-126): the
    bundled input projection holds the signal rows (left | right) then the gate rows (left | right); the transition's
    w12 holds the SwiGLU's two halves one behind the other (tt_bio/esmc.py:213-219)."""
    out: Dict[str, torch.Tensor] = {}
    for name in ("tri_mul_out", "tri_mul_in"):
        e = _sub(sd, f"{name}._engine")
        bundle = e["proj_bundle.weight"]
        half = bundle.shape[0] // 2
        out.update({
            f"{name}.norm_in.weight": e["norm_start.weight"], f"{name}.norm_in.bias": e["norm_start.bias"],
            f"{name}.norm_out.weight": e["norm_mix.weight"], f"{name}.norm_out.bias": e["norm_mix.bias"],
            f"{name}.p_in.weight": bundle[:half], f"{name}.g_in.weight": bundle[half:],
            f"{name}.p_out.weight": e["proj_emit.weight"], f"{name}.g_out.weight": e["proj_gate.weight"],
        })
    w12 = sd["pair_transition.ffn.w12.weight"]
    hidden = w12.shape[0] // 2
    out.update({
        "transition_z.norm.weight": sd["pair_transition.norm.weight"], "transition_z.norm.bias": sd["pair_transition.norm.bias"],
        "transition_z.fc1.weight": w12[:hidden], "transition_z.fc2.weight": w12[hidden:],
        "transition_z.fc3.weight": sd["pair_transition.ffn.w3.weight"],
    })
    return out
