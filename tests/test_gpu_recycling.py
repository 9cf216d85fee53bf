"""The resident recycling loop (tt_bio/boltz2.py:5203-5250) on the GPU against a CPU restatement that uses the
oracle for the Pairformer passes."""
import pytest
import torch
import torch.nn.functional as F

from oracle import pairformer_oracle as orc
from tests.conftest import rel_l2
from tt_boltz_b200 import B200PairformerModule, B200RecyclingTrunk, _lib, synthetic

pytestmark = pytest.mark.gpu


def _cpu_loop(w, sd, blocks, s_init, z_init, m, pm, steps, pair_update=None):
    s, z = torch.zeros_like(s_init), torch.zeros_like(z_init)
    for _ in range(steps + 1):
        s = s_init + F.layer_norm(s, (s.shape[-1],), w["s_norm.weight"], w["s_norm.bias"]) @ w["s_recycle.weight"].T
        z = z_init + F.layer_norm(z, (z.shape[-1],), w["z_norm.weight"], w["z_norm.bias"]) @ w["z_recycle.weight"].T
        if pair_update is not None:
            z = z + pair_update(z)
        s, z = orc.pairformer_stack(s, z, m, pm, sd, blocks)
    return s, z


@pytest.mark.parametrize("precision,tol", [("fp32", 2e-4), ("bf16", 2e-2)])
def test_recycling_loop_matches_cpu_restatement(precision, tol):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    n, blocks, steps = 40, 2, 2
    sd = synthetic.make_weights(blocks, seed=1, std=0.05, affine_jitter=0.2)
    s_init, z_init = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 5)
    g = torch.Generator().manual_seed(21)
    w = {"s_norm.weight": 1 + 0.2 * torch.randn(384, generator=g), "s_norm.bias": 0.2 * torch.randn(384, generator=g),
         "z_norm.weight": 1 + 0.2 * torch.randn(128, generator=g), "z_norm.bias": 0.2 * torch.randn(128, generator=g),
         "s_recycle.weight": 0.05 * torch.randn(384, 384, generator=g), "z_recycle.weight": 0.08 * torch.randn(128, 128, generator=g)}
    trunk = B200RecyclingTrunk(B200PairformerModule(384, 128, blocks, v2=True, precision=precision))
    state = dict(w)
    state.update({"pairformer_module." + k: v for k, v in sd.items()})
    trunk.load_state_dict(state, strict=True)              # the reference's key names, one flat dict
    update = lambda z: 0.05 * torch.tanh(z)                # stands for the template / MSA modules between the two
    for hook in (None, update):
        so, zo = trunk(s_init.to(dev), z_init.to(dev), m.to(dev), pm.to(dev), recycling_steps=steps, pair_update=hook)
        assert _lib.device_status() == 0
        with torch.no_grad():
            sr, zr = _cpu_loop(w, sd, blocks, s_init[0], z_init[0], m[0], pm[0], steps, hook)
        v = n - 5
        assert rel_l2(zo[0].cpu()[:v, :v], zr[:v, :v]) < tol, (precision, hook is not None)
        assert rel_l2(so[0].cpu()[:v], sr[:v]) < tol, (precision, hook is not None)
    # zero recycles = one pass from s = z = 0: LayerNorm of zeros is its offset
    so, zo = trunk(s_init.to(dev), z_init.to(dev), m.to(dev), pm.to(dev), recycling_steps=0)
    with torch.no_grad():
        sr, zr = _cpu_loop(w, sd, blocks, s_init[0], z_init[0], m[0], pm[0], 0)
    assert rel_l2(zo[0].cpu()[:35, :35], zr[:35, :35]) < tol


def test_distogram_head_against_the_reference_module():
    """tests/golden/heads/distogram_n12.npz: the reference's DistogramModule on a non-symmetric z (fp32 tier: 1e-5)."""
    import os
    import numpy as np
    from tt_boltz_b200 import B200DistogramModule
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "heads", "distogram_n12.npz"))
    head = B200DistogramModule(128, 64)
    head.load_state_dict({k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("w::")}, strict=True)
    z = torch.from_numpy(g["z"])
    got = head.cuda()(z.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert got.shape == (1, 12, 12, 1, 64)
    assert rel_l2(got.cpu(), torch.from_numpy(g["out"])) < 1e-5
