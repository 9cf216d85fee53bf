"""Parity at the sizes the benchmark times, against the reference's own CPU modules.

One reference block at N = 1024 costs half a minute of CPU and a z of 512 MiB, so the comparison uses the
committed sampled fixtures of tests/golden/sampled/ (made once by tests/golden/make_sampled_trunk.py from
``tt_bio.reference.PairformerModule``: z at 65 536 fixed positions, the whole of s, after 1, 8 and 64 blocks of
the benchmark's own inputs and weights).  Tolerances are the tiers': bf16 2e-2 (after 64 blocks too), MXFP8 5e-2.
"""
import os

import numpy as np
import pytest
import torch

from oracle import pairformer_oracle as orc
from tests.conftest import rel_l2
from tests.golden.make_golden import weight_checksum
from tt_boltz_b200 import B200PairformerModule, _lib, synthetic

pytestmark = pytest.mark.gpu
SAMPLED = os.path.join(os.path.dirname(__file__), "golden", "sampled")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def _fixture(name):
    path = os.path.join(SAMPLED, name)
    assert os.path.exists(path), f"{path} is missing (tests/golden/make_sampled_trunk.py writes it)"
    return np.load(path)


@pytest.mark.parametrize("precision,tol", [("bf16", 2e-2), ("mxfp8", 5e-2)])
def test_trunk_n1024_64_blocks_against_reference_samples(dev, precision, tol):
    """cfg-4 as the benchmark runs it: N = 1024, 64 blocks, all-ones masks, seeds 0 / 1.  Checked after 1, 8 and
    64 blocks, so that a defect that only shows with 8 query tiles, 16 key tiles or all SMs busy is caught at
    the first block and error growth over the depth at the last."""
    fx = _fixture("trunk_n1024_b64.npz")
    n, nb = int(fx["n"]), int(fx["blocks"])
    sd = synthetic.make_weights(nb, seed=1)
    assert abs(weight_checksum(sd) - float(fx["weight_checksum"])) <= 1e-6 * float(fx["weight_checksum"])
    s, z = synthetic.make_inputs(n, seed=0)
    assert np.array_equal(z.reshape(-1)[torch.from_numpy(fx["index"])].numpy(), fx["z_in_samples"]), "inputs differ from the fixture's"
    m, pm = synthetic.tail_padding_mask(n, 0)
    mod = B200PairformerModule(384, 128, nb, v2=True, precision=precision)
    mod.load_state_dict(sd, strict=True)
    del sd
    s_d, z_d, m_d, pm_d = s.to(dev), z.to(dev), m.to(dev), pm.to(dev)
    all_layers = list(mod.layers)
    done = 0
    for blocks in [int(b) for b in fx["snapshots"]]:
        # continue from the previous snapshot: the module's own forward over the next slice of layers
        mod.layers = torch.nn.ModuleList(all_layers[done:blocks])
        s_d, z_d = mod(s_d, z_d, m_d, pm_d)
        done = blocks
        assert _lib.device_status() == 0
        rz, rs = synthetic.sampled_fixture_errors(fx, blocks, s_d[0], z_d[0])
        limit = tol if blocks > 1 else tol / 4          # one block has no depth to hide behind
        assert rz < limit and rs < limit, (precision, blocks, rz, rs)
        norm = float(z_d.double().norm())
        assert abs(norm - float(fx[f"z_norm_{blocks}"])) < 2 * tol * float(fx[f"z_norm_{blocks}"])


@pytest.mark.parametrize("precision,tol", [("bf16", 2e-2), ("mxfp8", 5e-2)])
def test_cfg5_shape_random_padding_against_oracle(dev, precision, tol):
    """The large-complex configuration's ingredients at a size the oracle finishes in seconds: 5 % of the tokens
    masked AT RANDOM (seed 3, not a tail), several blocks, the MXFP8 tier; every key tile then holds masked keys."""
    n, nb = 256, 4
    sd = synthetic.make_weights(nb, seed=1)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.random_padding_mask(n, 0.05, seed=3)
    assert 0 < int((m == 0).sum()) < n // 8
    mod = B200PairformerModule(384, 128, nb, v2=True, precision=precision)
    mod.load_state_dict(sd, strict=True)
    so, zo = mod(s.to(dev), z.to(dev), m.to(dev), pm.to(dev))
    assert _lib.device_status() == 0
    with torch.no_grad():
        sr, zr = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, nb)
    keep = m[0].bool()
    assert rel_l2(zo[0].cpu()[keep][:, keep], zr[keep][:, keep]) < tol
    assert rel_l2(so[0].cpu()[keep], sr[keep]) < tol
    # what is stored at the masked tokens must not reach the valid region, bit for bit
    g = torch.Generator().manual_seed(17)
    z2, s2 = z.clone(), s.clone()
    z2[0, ~keep] = 20 * torch.randn(z2[0, ~keep].shape, generator=g)
    z2[0, :, ~keep] = 20 * torch.randn(z2[0, :, ~keep].shape, generator=g)
    s2[0, ~keep] = 20 * torch.randn(s2[0, ~keep].shape, generator=g)
    so2, zo2 = mod(s2.to(dev), z2.to(dev), m.to(dev), pm.to(dev))
    assert torch.equal(zo2[0][keep][:, keep], zo[0][keep][:, keep])
    assert torch.equal(so2[0][keep], so[0][keep])


def test_block_n2048_random_padding_against_reference_samples(dev):
    """One block of the large-complex configuration at its own size (N = 2048, 5 % random padding, MXFP8
    triangle multiplication) against the sampled reference fixture, when that fixture has been generated."""
    path = os.path.join(SAMPLED, "trunk_n2048_b1_pad.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/sampled/trunk_n2048_b1_pad.npz not generated")
    fx = np.load(path)
    n = int(fx["n"])
    sd = synthetic.make_weights(1, seed=1)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.random_padding_mask(n, float(fx["pad_frac"]), seed=3)
    assert np.array_equal(m[0].numpy(), fx["mask"])
    for precision, tol in (("mxfp8", 5e-2 / 4), ("bf16", 2e-2 / 4)):
        mod = B200PairformerModule(384, 128, 1, v2=True, precision=precision)
        mod.load_state_dict(sd, strict=True)
        so, zo = mod(s.to(dev), z.to(dev), m.to(dev), pm.to(dev))
        assert _lib.device_status() == 0
        # sampled positions that fall on masked tokens are not comparable (the reference leaves them unspecified)
        idx = torch.from_numpy(fx["index"])
        i, j = idx // (n * 128), (idx // 128) % n
        ok = (m[0][i] * m[0][j]).bool()
        z_ref = torch.from_numpy(fx["z_samples_1"])[ok].double()
        z_got = zo[0].reshape(-1)[idx.to(dev)].cpu()[ok].double()
        keep = m[0].bool()
        rz = float((z_got - z_ref).norm() / z_ref.norm())
        rs = rel_l2(so[0].cpu()[keep], torch.from_numpy(fx["s_1"])[keep])
        assert rz < tol and rs < tol, (precision, rz, rs)
        del mod, so, zo
