"""The CPU oracle must reproduce the outputs of the reference's own CPU Pairformer.

Fixtures: tests/golden/*.npz, written by tests/golden/make_golden.py from
tt_bio.reference.PairformerModule / PairformerNoSeqModule (fp32, eval, use_kernels=False).
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import msa_oracle
from oracle import pairformer_oracle as orc
from tests.golden.make_golden import weight_checksum
from tt_boltz_b200 import synthetic
from tests.conftest import rel_l2

CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
OPM_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "msa", "opm_*.npz")))


def load_case(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    n, nb, with_s = int(g["n"]), int(g["blocks"]), bool(g["with_s"])
    sd = synthetic.make_weights(nb, seed=1, std=float(g["std"]), affine_jitter=float(g["jitter"]), with_s=with_s)
    assert abs(weight_checksum(sd) - float(g["weight_checksum"])) <= 1e-6 * float(g["weight_checksum"]), \
        "regenerated weights differ from the ones the fixture was made with"
    s, z = synthetic.make_inputs(n, seed=0, with_s=with_s)
    return g, sd, s, z, torch.from_numpy(g["mask"]), torch.from_numpy(g["pair_mask"])


def test_fixtures_present():
    assert len(CASES) >= 5


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_outputs(golden_dir, name):
    g, sd, s, z, m, pm = load_case(golden_dir, name)
    with torch.no_grad():
        s_o, z_o = orc.pairformer_stack(None if s is None else s[0], z[0], m[0], pm[0], sd, int(g["blocks"]))
    assert rel_l2(z_o, torch.from_numpy(g["z_out"])[0]) < 2e-6
    if s is not None:
        assert rel_l2(s_o, torch.from_numpy(g["s_out"])[0]) < 2e-6


def test_oracle_sub_op_taps(golden_dir):
    g, sd, s, z, m, pm = load_case(golden_dir, "layer_n16_taps")
    taps = {}
    with torch.no_grad():
        orc.pairformer_layer(s[0], z[0], m[0], pm[0], sd, "layers.0.", taps=taps)
    for k in ("tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end", "transition_z"):
        assert rel_l2(taps[k], torch.from_numpy(g["tap_" + k])[0]) < 2e-6, k


def test_oracle_padding_isolated(golden_dir):
    """Values stored at masked-out tokens must not leak into the valid region (exactly)."""
    g, sd, s, z, m, pm = load_case(golden_dir, "stack2_n20_tailpad")
    gen = torch.Generator().manual_seed(11)
    z2, s2 = z.clone(), s.clone()
    pad = (m[0] == 0)
    z2[0, pad] = 50 * torch.randn(z2[0, pad].shape, generator=gen)
    z2[0, :, pad] = 50 * torch.randn(z2[0, :, pad].shape, generator=gen)
    s2[0, pad] = 50 * torch.randn(s2[0, pad].shape, generator=gen)
    with torch.no_grad():
        sa, za = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, 2)
        sb, zb = orc.pairformer_stack(s2[0], z2[0], m[0], pm[0], sd, 2)
    v = ~pad
    assert torch.equal(za[v][:, v], zb[v][:, v])
    assert torch.equal(sa[v], sb[v])
    assert torch.isfinite(zb).all() and torch.isfinite(sb).all()


@pytest.mark.parametrize("name", OPM_CASES)
def test_outer_product_mean_oracle_matches_reference_outputs(golden_dir, name):
    """tests/golden/msa/make_opm.py stored what tt_bio.reference.OuterProductMean returns (both of its branches)."""
    g = np.load(os.path.join(golden_dir, "msa", name + ".npz"))
    w = synthetic.make_opm_weights(seed=int(g["weight_seed"]))
    m, mask = synthetic.make_msa_inputs(int(g["s"]), int(g["n"]), drop=float(g["drop"]), seed=int(g["input_seed"]))
    with torch.no_grad():
        out = msa_oracle.outer_product_mean(m, mask, w)
    assert rel_l2(out, torch.from_numpy(g["out"])) < 2e-6


def test_outer_product_mean_fixtures_present():
    assert len(OPM_CASES) >= 3


MSA_LAYER_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "msa", "msa_layer_*.npz")))


def load_msa_layer_case(golden_dir, name):
    from tests.golden.msa.make_msa_layer import make_case_inputs
    g = np.load(os.path.join(golden_dir, "msa", name + ".npz"))
    c = dict(s=int(g["s"]), n=int(g["n"]), drop=float(g["drop"]), pad=int(g["pad"]))
    return g, synthetic.make_msa_layer_weights(seed=int(g["weight_seed"])), make_case_inputs(c)


@pytest.mark.parametrize("name", MSA_LAYER_CASES)
def test_msa_layer_oracle_matches_reference_outputs(golden_dir, name):
    """tests/golden/msa/make_msa_layer.py stored what tt_bio.reference.MSALayer and its sub-modules return."""
    g, w, (z, m, token_mask, msa_mask) = load_msa_layer_case(golden_dir, name)
    with torch.no_grad():
        pwa = msa_oracle.pair_weighted_averaging(m, z, token_mask, msa_oracle._sub(w, "pair_weighted_averaging."))
        trans = msa_oracle.msa_transition(m, msa_oracle._sub(w, "msa_transition."))
        z_o, m_o = msa_oracle.msa_layer(z, m, token_mask, msa_mask, w)
    assert rel_l2(pwa, torch.from_numpy(g["pwa"])) < 2e-6
    assert rel_l2(trans, torch.from_numpy(g["transition"])) < 2e-6
    assert rel_l2(m_o, torch.from_numpy(g["m_out"])) < 2e-6
    assert rel_l2(z_o, torch.from_numpy(g["z_out"])) < 2e-6


def test_msa_layer_fixtures_present():
    assert len(MSA_LAYER_CASES) >= 2


def test_msa_module_oracle_matches_reference_output(golden_dir):
    """tests/golden/msa/make_msa_module.py stored what tt_bio.reference.MSAModule.forward returns."""
    from tests.golden.msa.make_msa_module import make_case_inputs
    g = np.load(os.path.join(golden_dir, "msa", "msa_module_s9_n21.npz"))
    c = dict(s=int(g["s"]), n=int(g["n"]), blocks=int(g["blocks"]), pad=int(g["pad"]))
    z, emb, feats = make_case_inputs(c)
    with torch.no_grad():
        out = msa_oracle.msa_module(z[0], emb[0], feats, synthetic.make_msa_module_weights(c["blocks"]), c["blocks"])
    assert rel_l2(out, torch.from_numpy(g["z_out"])) < 2e-6


WIDTH_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "widths", "*.npz")))


def load_width_case(golden_dir, name):
    """Fixtures of tests/golden/widths/make_widths.py: the reference's modules at pair widths 64 and 256."""
    g = np.load(os.path.join(golden_dir, "widths", name + ".npz"))
    n, nb, with_s, c_z, heads = int(g["n"]), int(g["blocks"]), bool(g["with_s"]), int(g["c_z"]), int(g["tri_heads"])
    sd = synthetic.make_weights(nb, seed=1, std=float(g["std"]), affine_jitter=float(g["jitter"]), with_s=with_s, c_z=c_z, tri_heads=heads)
    assert abs(weight_checksum(sd) - float(g["weight_checksum"])) <= 1e-6 * float(g["weight_checksum"]), \
        "regenerated weights differ from the ones the fixture was made with"
    s, z = synthetic.make_inputs(n, c_z=c_z, seed=0, with_s=with_s)
    return g, sd, s, z, torch.from_numpy(g["mask"]), torch.from_numpy(g["pair_mask"])


@pytest.mark.parametrize("name", WIDTH_CASES)
def test_oracle_matches_reference_outputs_at_other_widths(golden_dir, name):
    """The template stack (c_z = 64) and a c_z = 256 / eight-head block: the oracle is generic in the widths and is
    pinned to the reference's own modules there too."""
    g, sd, s, z, m, pm = load_width_case(golden_dir, name)
    assert len(WIDTH_CASES) >= 2
    with torch.no_grad():
        s_o, z_o = orc.pairformer_stack(None if s is None else s[0], z[0], m[0], pm[0], sd, int(g["blocks"]))
    assert rel_l2(z_o, torch.from_numpy(g["z_out"])[0]) < 2e-6
    if s is not None:
        assert rel_l2(s_o, torch.from_numpy(g["s_out"])[0]) < 2e-6
