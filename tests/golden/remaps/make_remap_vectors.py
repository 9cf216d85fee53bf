"""Generate the sibling-model fixtures in this folder from the reference's own code.

Run where the reference checkout is importable:

    python tests/golden/remaps/make_remap_vectors.py --reference /path/to/tt-boltz

Two kinds of fixture:

* ``esmfold2_block_*.npz``: one block of the ESMFold2 folding trunk, computed by the reference's vendored PyTorch
  model (``tt_bio/_vendor/esmfold2_hf/modeling_esmfold2_common.py`` ``PairUpdateBlock``: outgoing and incoming
  triangle multiplication with the bundled input projection, then the SwiGLU transition with its residual) in fp32 on
  the CPU, with every parameter overwritten by seeded values.  Stored: the block's state dict under ITS key names,
  the pair tensor, the pair mask and the output.
* ``protenix_remaps.npz``: what the reference's own remap functions (``tt_bio/protenix_weights.py``
  ``remap_pairformer_block``, ``remap_msa_pair_stack``, ``remap_outer_product_mean``,
  ``remap_pair_weighted_averaging``) return for state dicts written under the Protenix / OpenFold key names.  The
  tensors are tiny and every element is distinct (a per-tensor offset plus a running index), so that a wrong source
  key, a swapped concatenation order or a wrong row split cannot give the same values.

``ttnn`` (a device library, the one missing import of the reference package) is replaced by a stub.
"""
from __future__ import annotations

import argparse
import os
import sys
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

ESMFOLD2_CASES = {
    # name: width, tokens, padded tail tokens, general (non-outer-product) mask
    "esmfold2_block_c64_n14": dict(c=64, n=14, pad=3, general=False),
    "esmfold2_block_c32_n9_general_mask": dict(c=32, n=9, pad=0, general=True),
}

# Key names of one Protenix PairformerBlock (tt_bio/protenix_weights.py:17-93 reads exactly these), with row counts
# per tensor small enough for a fixture of a few KB: (name, shape)
C_Z, C_S, HID, HEADS = 6, 8, 4, 2


def protenix_block_keys(with_s: bool):
    keys = []
    for name in ("tri_mul_out", "tri_mul_in"):
        keys += [(f"{name}.layer_norm_in.weight", (C_Z,)), (f"{name}.layer_norm_in.bias", (C_Z,)),
                 (f"{name}.layer_norm_out.weight", (HID,)), (f"{name}.layer_norm_out.bias", (HID,)),
                 (f"{name}.linear_a_g.weight", (HID, C_Z)), (f"{name}.linear_b_g.weight", (HID, C_Z)),
                 (f"{name}.linear_a_p.weight", (HID, C_Z)), (f"{name}.linear_b_p.weight", (HID, C_Z)),
                 (f"{name}.linear_g.weight", (C_Z, C_Z)), (f"{name}.linear_z.weight", (C_Z, HID))]
    for name in ("tri_att_start", "tri_att_end"):
        keys += [(f"{name}.layer_norm.weight", (C_Z,)), (f"{name}.layer_norm.bias", (C_Z,)),
                 (f"{name}.linear.weight", (HEADS, C_Z))]
        keys += [(f"{name}.mha.linear_{x}.weight", (HID, C_Z)) for x in ("q", "k", "v", "g")]
        keys += [(f"{name}.mha.linear_o.weight", (C_Z, HID))]
    keys += [("pair_transition.layernorm1.weight", (C_Z,)), ("pair_transition.layernorm1.bias", (C_Z,)),
             ("pair_transition.linear_no_bias_a.weight", (2 * C_Z, C_Z)), ("pair_transition.linear_no_bias_b.weight", (2 * C_Z, C_Z)),
             ("pair_transition.linear_no_bias.weight", (C_Z, 2 * C_Z))]
    if with_s:
        p = "attention_pair_bias."
        keys += [(p + "layernorm_a.weight", (C_S,)), (p + "layernorm_a.bias", (C_S,)),
                 (p + "attention.linear_q.weight", (C_S, C_S)), (p + "attention.linear_q.bias", (C_S,))]
        keys += [(p + f"attention.linear_{x}.weight", (C_S, C_S)) for x in ("k", "v", "g", "o")]
        keys += [(p + "layernorm_z.weight", (C_Z,)), (p + "layernorm_z.bias", (C_Z,)), (p + "linear_nobias_z.weight", (HEADS, C_Z))]
        keys += [("single_transition.layernorm1.weight", (C_S,)), ("single_transition.layernorm1.bias", (C_S,)),
                 ("single_transition.linear_no_bias_a.weight", (2 * C_S, C_S)), ("single_transition.linear_no_bias_b.weight", (2 * C_S, C_S)),
                 ("single_transition.linear_no_bias.weight", (C_S, 2 * C_S))]
    return keys


OPM_KEYS = [("layer_norm.weight", (C_S,)), ("layer_norm.bias", (C_S,)), ("linear_1.weight", (HID, C_S)), ("linear_2.weight", (HID, C_S)),
            ("linear_out.weight", (C_Z, HID * HID)), ("linear_out.bias", (C_Z,))]
PWA_KEYS = [("layernorm_m.weight", (C_S,)), ("layernorm_m.bias", (C_S,)), ("layernorm_z.weight", (C_Z,)), ("layernorm_z.bias", (C_Z,)),
            ("linear_no_bias_mv.weight", (HID * HEADS, C_S)), ("linear_no_bias_mg.weight", (HID * HEADS, C_S)),
            ("linear_no_bias_z.weight", (HEADS, C_Z)), ("linear_no_bias_out.weight", (C_S, HID * HEADS))]


def coded(keys):
    """Every element distinct across the whole dict: tensor t holds 1000 t + 0, 1, 2, ..."""
    return {k: (1000.0 * i + torch.arange(int(np.prod(shape)), dtype=torch.float32)).reshape(shape) for i, (k, shape) in enumerate(keys)}


def seeded_block_weights(state, seed):
    """Seeded values for every parameter of the block (its own initialisation zeroes some gates)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for k, v in state.items():
        if k.endswith("norm_start.weight") or k.endswith("norm_mix.weight") or k.endswith("norm.weight"):
            out[k] = 1 + 0.2 * torch.randn(v.shape, generator=g)
        elif k.endswith(".bias"):
            out[k] = 0.2 * torch.randn(v.shape, generator=g)
        else:
            out[k] = torch.randn(v.shape, generator=g) / float(v.shape[-1]) ** 0.5
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a tt-boltz checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.modules.setdefault("ttnn", MagicMock(name="ttnn"))
    import importlib
    hf = importlib.import_module("tt_bio._vendor.esmfold2_hf.modeling_esmfold2_common")
    pw = importlib.import_module("tt_bio.protenix_weights")

    torch.set_grad_enabled(False)
    for name, c in ESMFOLD2_CASES.items():
        blk = hf.PairUpdateBlock(d_pair=c["c"], expansion_ratio=4).eval()
        w = seeded_block_weights(blk.state_dict(), seed=17)
        blk.load_state_dict(w, strict=True)
        g = torch.Generator().manual_seed(23)
        n = c["n"]
        z = torch.randn(1, n, n, c["c"], generator=g)
        if c["general"]:
            mask = (torch.rand(1, n, n, generator=g) > 0.3).float()
        else:
            tok = torch.ones(n)
            tok[n - c["pad"]:] = 0
            mask = (tok[:, None] * tok[None, :])[None]
        out = blk(z, pair_attention_mask=mask)
        arrays = {"w::" + k: v.numpy() for k, v in w.items()}
        np.savez_compressed(os.path.join(HERE, name + ".npz"), z=z.numpy(), mask=mask.numpy(), out=out.numpy().astype(np.float32), **arrays)
        print(name, tuple(out.shape), float(out.abs().mean()))

    arrays = {}
    for tag, keys, fn in (("block", protenix_block_keys(True), pw.remap_pairformer_block),
                          ("pair_stack", protenix_block_keys(False), pw.remap_msa_pair_stack),
                          ("opm", OPM_KEYS, pw.remap_outer_product_mean),
                          ("pwa", PWA_KEYS, pw.remap_pair_weighted_averaging)):
        theirs = coded(keys)
        mapped = fn(theirs)
        for k, v in theirs.items():
            arrays[f"{tag}::in::{k}"] = v.numpy()
        for k, v in mapped.items():
            arrays[f"{tag}::out::{k}"] = v.numpy()
        print(tag, len(theirs), "->", len(mapped), "tensors")
    # the pair-bias LayerNorm may come without an offset: the reference then supplies zeros
    theirs = coded(protenix_block_keys(True))
    del theirs["attention_pair_bias.layernorm_z.bias"]
    arrays["block_no_z_bias::out::attention.proj_z.0.bias"] = pw.remap_pairformer_block(theirs)["attention.proj_z.0.bias"].numpy()
    np.savez_compressed(os.path.join(HERE, "protenix_remaps.npz"), **arrays)


if __name__ == "__main__":
    main()
