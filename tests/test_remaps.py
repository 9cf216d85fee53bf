"""Checkpoint key remaps of the sibling models (tt_bio/protenix_weights.py:17-137, tt_bio/esmfold2.py:102-126): a
checkpoint written with THEIR key names must load, strictly, into our modules and give back the same tensors."""
import torch

from tt_boltz_b200 import B200OuterProductMean, B200PairformerModule, B200PairformerNoSeqLayer, B200PairUpdateBlock, remaps, synthetic

DIMS = dict(c_s=384, c_z=256, num_heads=16, tri_heads=8, tri_head_dim=32)


def _invert(ours, table, prefix_ours, prefix_theirs):
    """Write OUR tensors under THEIR names (splitting concatenated rows back into their parts)."""
    out = {}
    for k_ours, src in table.items():
        t = ours[prefix_ours + k_ours]
        if isinstance(src, tuple):
            for part, name in zip(torch.chunk(t, len(src), dim=0), src):
                out[prefix_theirs + name] = part
        else:
            out[prefix_theirs + src] = t
    return out


def _protenix_block_from_ours(ours, with_s):
    theirs = {}
    for name in ("tri_mul_out", "tri_mul_in"):
        theirs.update(_invert(ours, remaps.TRIANGLE_MULTIPLICATION, name + ".", name + "."))
    for k, v in ours.items():
        if k.startswith("tri_att_"):
            theirs[k] = v
    theirs.update(_invert(ours, remaps.TRANSITION, "transition_z.", "pair_transition."))
    if with_s:
        theirs.update(_invert(ours, remaps.ATTENTION_PAIR_BIAS, "attention.", "attention_pair_bias."))
        theirs["attention_pair_bias.layernorm_a.weight"] = ours["pre_norm_s.weight"]
        theirs["attention_pair_bias.layernorm_a.bias"] = ours["pre_norm_s.bias"]
        theirs.update(_invert(ours, remaps.TRANSITION, "transition_s.", "single_transition."))
    return theirs


def test_protenix_pairformer_block_round_trip_and_strict_load():
    ours = {k[len("layers.0."):]: v for k, v in synthetic.make_weights(1, affine_jitter=0.1, **DIMS).items()}
    theirs = _protenix_block_from_ours(ours, with_s=True)
    assert not any(k.startswith(("transition_z.", "attention.", "pre_norm_s")) for k in theirs)
    back = remaps.protenix_pairformer_block(theirs)
    assert set(back) == set(ours)
    for k in ours:
        assert torch.equal(back[k], ours[k]), k
    mod = B200PairformerModule(384, 256, 1, pairwise_num_heads=8, precision="auto")
    assert mod.layers[0].precision == "fp32"
    mod.load_state_dict({"layers.0." + k: v for k, v in back.items()}, strict=True)
    # a LayerNorm on the pair bias without an offset in the source becomes a zero offset
    del theirs["attention_pair_bias.layernorm_z.bias"]
    assert torch.count_nonzero(remaps.protenix_pairformer_block(theirs)["attention.proj_z.0.bias"]) == 0


def test_protenix_pair_stack_and_outer_product_mean():
    ours = {k[len("layers.0."):]: v for k, v in synthetic.make_weights(1, with_s=False, c_z=128).items()}
    back = remaps.protenix_pair_stack(_protenix_block_from_ours(ours, with_s=False))
    B200PairformerNoSeqLayer(128).load_state_dict(back, strict=True)
    opm = synthetic.make_opm_weights()
    theirs = _invert(opm, remaps.OUTER_PRODUCT_MEAN, "", "")
    B200OuterProductMean().load_state_dict(remaps.protenix_outer_product_mean(theirs), strict=True)


def test_esmfold2_pair_update_block():
    c, hidden = 256, 512
    blk = B200PairUpdateBlock(c, hidden)
    g = torch.Generator().manual_seed(0)
    ours = {k: torch.randn(v.shape, generator=g) for k, v in blk.state_dict().items()}
    theirs = {}
    for name in ("tri_mul_out", "tri_mul_in"):
        e = f"{name}._engine."
        theirs[e + "proj_bundle.weight"] = torch.cat([ours[f"{name}.p_in.weight"], ours[f"{name}.g_in.weight"]], 0)
        for a, b in (("norm_in", "norm_start"), ("norm_out", "norm_mix")):
            theirs[e + b + ".weight"], theirs[e + b + ".bias"] = ours[f"{name}.{a}.weight"], ours[f"{name}.{a}.bias"]
        theirs[e + "proj_emit.weight"], theirs[e + "proj_gate.weight"] = ours[f"{name}.p_out.weight"], ours[f"{name}.g_out.weight"]
    theirs["pair_transition.norm.weight"], theirs["pair_transition.norm.bias"] = ours["transition_z.norm.weight"], ours["transition_z.norm.bias"]
    theirs["pair_transition.ffn.w12.weight"] = torch.cat([ours["transition_z.fc1.weight"], ours["transition_z.fc2.weight"]], 0)
    theirs["pair_transition.ffn.w3.weight"] = ours["transition_z.fc3.weight"]
    back = remaps.esmfold2_pair_update_block(theirs)
    blk.load_state_dict(back, strict=True)
    for k in ours:
        assert torch.equal(back[k], ours[k]), k


# ---- pinned against the reference's own code (fixtures written by tests/golden/remaps/make_remap_vectors.py) ----

import glob
import os

import numpy as np
import pytest

REMAP_DIR = os.path.join(os.path.dirname(__file__), "golden", "remaps")
ESMFOLD2_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(REMAP_DIR, "esmfold2_block_*.npz")))


def _tagged(g, tag, side):
    pre = f"{tag}::{side}::"
    return {k[len(pre):]: torch.from_numpy(g[k]) for k in g.files if k.startswith(pre)}


@pytest.mark.parametrize("tag, fn", [("block", remaps.protenix_pairformer_block), ("pair_stack", remaps.protenix_pair_stack),
                                     ("opm", remaps.protenix_outer_product_mean), ("pwa", remaps.protenix_pair_weighted_averaging)])
def test_protenix_remaps_reproduce_the_reference_functions(tag, fn):
    """tt_bio/protenix_weights.py remap_pairformer_block / remap_msa_pair_stack / remap_outer_product_mean /
    remap_pair_weighted_averaging were run on state dicts whose every element is distinct; ours must return the same
    keys with the same tensors (source key, concatenation order and row order all show in the values)."""
    g = np.load(os.path.join(REMAP_DIR, "protenix_remaps.npz"))
    theirs, want = _tagged(g, tag, "in"), _tagged(g, tag, "out")
    assert len(theirs) > 0 and len(want) > 0
    got = fn(theirs)
    assert set(got) == set(want)
    for k in want:
        assert got[k].shape == want[k].shape and torch.equal(got[k], want[k]), k


def test_protenix_pair_bias_norm_without_offset_matches_the_reference():
    g = np.load(os.path.join(REMAP_DIR, "protenix_remaps.npz"))
    theirs = _tagged(g, "block", "in")
    del theirs["attention_pair_bias.layernorm_z.bias"]
    want = torch.from_numpy(g["block_no_z_bias::out::attention.proj_z.0.bias"])
    assert torch.equal(remaps.protenix_pairformer_block(theirs)["attention.proj_z.0.bias"], want)


def load_esmfold2_case(name):
    g = np.load(os.path.join(REMAP_DIR, name + ".npz"))
    theirs = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("w::")}
    return theirs, torch.from_numpy(g["z"]), torch.from_numpy(g["mask"]), torch.from_numpy(g["out"])


@pytest.mark.parametrize("name", ESMFOLD2_CASES)
def test_esmfold2_block_through_our_remap_and_oracle_matches_the_reference_model(name):
    """The reference's vendored PyTorch ESMFold2 PairUpdateBlock (tt_bio/_vendor/esmfold2_hf/
    modeling_esmfold2_common.py) computed the stored output from weights under ITS names; the same weights through our
    remap and the CPU oracle's triangle multiplication and transition must give it back (fp32: 1e-5)."""
    from oracle import pairformer_oracle as orc
    theirs, z, mask, want = load_esmfold2_case(name)
    ours = remaps.esmfold2_pair_update_block(theirs)
    c = z.shape[-1]
    B200PairUpdateBlock(c, ours["transition_z.fc1.weight"].shape[0]).load_state_dict(ours, strict=True)
    with torch.no_grad():
        zz = z[0]
        zz = zz + orc.tri_mul(zz, ours, "tri_mul_out", mask[0], False)
        zz = zz + orc.tri_mul(zz, ours, "tri_mul_in", mask[0], True)
        zz = zz + orc.transition(zz, ours, "transition_z")
    err = ((zz - want[0]).norm() / want[0].norm()).item()
    assert err < 1e-5, err
