"""GPU parity of the outer-product mean (the MSA stack's write into the pair tensor) through the C ABI.

Checked against the committed outputs of the reference's own ``OuterProductMean`` (tests/golden/msa/opm_*.npz) and, at
sizes where blocks of tokens, ragged tiles and several mask words come into play, against the CPU oracle on the
same seeded inputs.  Tolerance: the bf16 tier's 2e-2 relative L2 (operands and both GEMM outputs are bf16, every
accumulation fp32); measured values are about 3e-3.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import msa_oracle
from tests.conftest import rel_l2
from tt_boltz_b200 import B200MSALayer, B200MSAModule, B200OuterProductMean, _lib, synthetic

pytestmark = pytest.mark.gpu
TOL = 2e-2

OPM_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "msa", "opm_*.npz")))


def _module(seed=11, **kw):
    mod = B200OuterProductMean(64, 32, 128, **kw)
    mod.load_state_dict(synthetic.make_opm_weights(seed=seed), strict=True)
    return mod.cuda()


@pytest.mark.parametrize("name", OPM_CASES)
def test_against_reference_fixture(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "msa", name + ".npz"))
    m, mask = synthetic.make_msa_inputs(int(g["s"]), int(g["n"]), drop=float(g["drop"]), seed=int(g["input_seed"]))
    out = _module(int(g["weight_seed"]))(m[None].cuda(), mask[None].cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(out[0].cpu(), torch.from_numpy(g["out"])) < TOL


@pytest.mark.parametrize("s_len, n, drop, block", [
    (200, 136, 0.3, None),        # ragged tiles in both GEMMs, 7 mask words
    (64, 260, 0.0, 24),           # several blocks of tokens with a short last one
    (1030, 48, 0.5, 20),          # more sequences than tokens, 33 mask words, heavy masking
])
def test_against_oracle(s_len, n, drop, block):
    m, mask = synthetic.make_msa_inputs(s_len, n, drop=drop, seed=9)
    w = synthetic.make_opm_weights(seed=3)
    with torch.no_grad():
        want = msa_oracle.outer_product_mean(m, mask, w)
    got = _module(3, block_tokens=block)(m[None].cuda(), mask[None].cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.isfinite(got).all()
    assert rel_l2(got[0].cpu(), want) < TOL


def test_pair_counts_are_exact():
    """With the projections replaced by constants the result is count-exact: every pair's mean of ones is one."""
    s_len, n = 70, 40
    m, mask = synthetic.make_msa_inputs(s_len, n, drop=0.5, seed=2)
    mask[:, 5] = 0                      # two tokens that no sequence covers: count 0, clamped to 1
    mask[:, 17] = 0
    w = synthetic.make_opm_weights(seed=3)
    # LN output = beta (gain 0); proj_a / proj_b pick a constant 1 in channel 0 -> a = b = mask * e0;
    # outer product sum = count * e0 e0^T; proj_o reads that entry with weight 1 -> count / max(count, 1)
    w["norm.weight"].zero_(); w["norm.bias"].fill_(1.0)
    for k in ("proj_a.weight", "proj_b.weight"):
        w[k].zero_(); w[k][0, 0] = 1.0
    w["proj_o.weight"].zero_(); w["proj_o.weight"][:, 0] = 1.0
    w["proj_o.bias"].zero_()
    mod = B200OuterProductMean(64, 32, 128)
    mod.load_state_dict(w, strict=True)
    got = mod.cuda()(m[None].cuda(), mask[None].cuda())[0].cpu()
    count = torch.einsum("si,sj->ij", mask, mask)
    want = (count > 0).float()[..., None].expand(n, n, 128)
    assert (count == 0).any() and (count > 1).any()
    assert torch.allclose(got, want, rtol=0, atol=2e-7)          # count * (1 / count) may be one ulp off 1
    assert torch.equal(got[count == 0], torch.zeros_like(got[count == 0]))


def test_add_into_accumulates_in_place():
    s_len, n = 40, 64
    m, mask = synthetic.make_msa_inputs(s_len, n, drop=0.2, seed=4)
    mod = _module()
    z = torch.randn(1, n, n, 128, generator=torch.Generator().manual_seed(1)).cuda()
    z0 = z.clone()
    upd = mod(m[None].cuda(), mask[None].cuda())
    ret = mod.add_into(z, m[None].cuda(), mask[None].cuda())
    assert ret is z
    assert torch.allclose(z, z0 + upd, rtol=0, atol=1e-5 * float(upd.abs().max()) + 1e-6)


# ---- the whole MSA layer: pair-weighted averaging, transition, outer-product mean, pair block ----
MSA_LAYER_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "msa", "msa_layer_*.npz")))


def _layer(seed=21):
    layer = B200MSALayer(64, 128, 0.0, 0.0)
    layer.load_state_dict(synthetic.make_msa_layer_weights(seed=seed), strict=True)
    return layer.cuda()


@pytest.mark.parametrize("name", MSA_LAYER_CASES)
def test_msa_layer_against_reference_fixture(golden_dir, name):
    from tests.test_oracle_golden import load_msa_layer_case
    g, _, (z, m, token_mask, msa_mask) = load_msa_layer_case(golden_dir, name)
    layer = _layer(int(g["weight_seed"]))
    zc, mc, tm, mm = z[None].cuda(), m[None].cuda(), token_mask[None].cuda(), msa_mask[None].cuda()
    pwa = layer.pair_weighted_averaging(mc, zc, tm)
    trans = layer.msa_transition(mc)
    z_o, m_o = layer(zc, mc, tm, mm)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(pwa[0].cpu(), torch.from_numpy(g["pwa"])) < TOL
    assert rel_l2(trans[0].cpu(), torch.from_numpy(g["transition"])) < TOL
    assert rel_l2(m_o[0].cpu(), torch.from_numpy(g["m_out"])) < TOL
    assert rel_l2(z_o[0].cpu(), torch.from_numpy(g["z_out"])) < TOL


def test_msa_layer_against_oracle_with_chunks(monkeypatch):
    """Sizes at which the sequence chunking, ragged GEMM tiles and the padded token axis all come into play."""
    from tt_boltz_b200 import msa as msa_mod
    monkeypatch.setattr(msa_mod, "ROWS_PER_CHUNK", 4096)          # 28 sequences of 144 padded tokens per chunk
    s_len, n = 75, 139
    _, z = synthetic.make_inputs(n, seed=6, with_s=False)
    m, msa_mask = synthetic.make_msa_inputs(s_len, n, drop=0.3, seed=7)
    _, pm = synthetic.random_padding_mask(n, 0.1, seed=3)
    w = synthetic.make_msa_layer_weights(seed=5)
    with torch.no_grad():
        z_want, m_want = msa_oracle.msa_layer(z[0], m, pm[0], msa_mask, w)
    z_o, m_o = _layer(5)(z.cuda(), m[None].cuda(), pm.cuda(), msa_mask[None].cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.isfinite(z_o).all() and torch.isfinite(m_o).all()
    assert rel_l2(m_o[0].cpu(), m_want) < TOL
    assert rel_l2(z_o[0].cpu(), z_want) < TOL


def test_msa_module_against_reference_fixture(golden_dir):
    """The whole MSA module (feature embedding + two blocks) against what tt_bio.reference.MSAModule returned."""
    from tests.golden.msa.make_msa_module import make_case_inputs
    g = np.load(os.path.join(golden_dir, "msa", "msa_module_s9_n21.npz"))
    c = dict(s=int(g["s"]), n=int(g["n"]), blocks=int(g["blocks"]), pad=int(g["pad"]))
    z, emb, feats = make_case_inputs(c)
    mod = B200MSAModule(64, 128, 384, c["blocks"], 0.0, 0.0)
    mod.load_state_dict(synthetic.make_msa_module_weights(c["blocks"]), strict=True)
    out = mod.cuda()(z.cuda(), emb.cuda(), {k: v.cuda() for k, v in feats.items()})
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(out[0].cpu(), torch.from_numpy(g["z_out"])) < TOL
