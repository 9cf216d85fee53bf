"""Host logic: weight packing and the module's state-dict surface, checked on the CPU.

The kernels cannot run here, so each packing layout is validated by a small torch model of what
the kernel does with the packed buffers (normalise without affine, multiply by the packed bf16
rows, add the folded bias, combine the values the layout puts side by side) against the oracle.
"""
import math

import pytest
import torch

from oracle import pairformer_oracle as orc
from tt_boltz_b200 import B200PairformerModule, B200PairformerNoSeqModule, synthetic, weights
from tests.conftest import rel_l2

N = 12


def xhat(z):
    mu = z.mean(-1, keepdim=True)
    var = ((z - mu) ** 2).mean(-1, keepdim=True)
    return (z - mu) * torch.rsqrt(var + 1e-5)


@pytest.fixture(scope="module")
def setup():
    sd = synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3)
    sd = {k[len("layers.0."):]: v for k, v in sd.items()}
    _, z = synthetic.make_inputs(N, seed=4)
    g = torch.Generator().manual_seed(9)
    pm = (torch.rand(N, N, generator=g) > 0.25).float()
    return sd, z[0], pm


@pytest.mark.parametrize("incoming", [False, True])
def test_trimul_packing_model(setup, incoming):
    sd, z, pm = setup
    pre = "tri_mul_in" if incoming else "tri_mul_out"
    pk = weights.pack_trimul(sd, pre + ".", "cpu")
    y = xhat(z) @ pk["w_pg"].float().T + pk["bias_pg"]            # [N,N,512]
    a = torch.empty(N, N, 128)
    b = torch.empty(N, N, 128)
    for q in range(8):
        ch = (q % 4) * 32
        u = y[..., q * 64:q * 64 + 32] * torch.sigmoid(y[..., q * 64 + 32:q * 64 + 64]) * pm[..., None]
        (a if q < 4 else b)[..., ch:ch + 32] = u
    t = torch.einsum("kic,kjc->ijc", a, b) if incoming else torch.einsum("ikc,jkc->ijc", a, b)
    upd = (xhat(t) @ pk["w_pout"].float().T + pk["bias_pout"]) * torch.sigmoid(xhat(z) @ pk["w_gout"].float().T + pk["bias_gout"])
    ref = orc.tri_mul(z, sd, pre, pm, incoming)
    assert rel_l2(upd, ref) < 1e-2


@pytest.mark.parametrize("ending", [False, True])
def test_triatt_packing_model(setup, ending):
    sd, z, pm = setup
    pre = "tri_att_end" if ending else "tri_att_start"
    pk = weights.pack_triatt(sd, pre + ".", "cpu")
    assert pk["w_qkvg"].shape == (528, 128) and pk["bias_qkvg"].shape == (528,)
    y = xhat(z) @ pk["w_qkvg"].float().T + pk["bias_qkvg"]        # [N,N,528] in z layout (r, c)
    if ending:          # line = column: (line, pos) = (c, r)
        y = y.transpose(0, 1)
        mask = pm.T
    else:
        mask = pm
    q, k, v = (y[..., i * 128:(i + 1) * 128].reshape(N, N, 4, 32) for i in range(3))
    gate = torch.sigmoid(y[..., 384:512])
    bias = y[..., 512:516]                                          # [line(q), pos(k), h], log2 domain
    s = torch.einsum("lqhd,lkhd->lhqk", q, k) + bias.permute(2, 0, 1)[None]
    s = torch.where(mask[:, None, None, :] > 0, s, torch.full_like(s, -1e9 * weights.LOG2E))
    p = torch.exp2(s - s.amax(-1, keepdim=True))
    p = p / p.sum(-1, keepdim=True)
    o = torch.einsum("lhqk,lkhd->lqhd", p, v).reshape(N, N, 128) * gate
    upd = o @ pk["w_o"].float().T
    if ending:
        upd = upd.transpose(0, 1)
    ref = orc.tri_att(z, sd, pre, pm, ending)
    assert rel_l2(upd, ref) < 1e-2


def test_transition_packing_model(setup):
    sd, z, _ = setup
    pk = weights.pack_transition_z(sd, "transition_z.", "cpu")
    assert pk["w12"].shape == (1024, 128) and pk["w3"].shape == (8, 128, 64)
    y = xhat(z) @ pk["w12"].float().T + pk["bias12"]               # [N,N,1024]
    out = torch.zeros(N, N, 128)
    for step in range(8):
        for sub in range(4):
            base = step * 128 + sub * 32
            f1, f2 = y[..., base:base + 16], y[..., base + 16:base + 32]
            h = torch.nn.functional.silu(f1) * f2
            out += h @ pk["w3"][step].float()[:, sub * 16:(sub + 1) * 16].T
    ref = orc.transition(z, sd, "transition_z")
    assert rel_l2(out, ref) < 1e-2


def test_module_state_dict_surface():
    sd = synthetic.make_weights(2, seed=1)
    m = B200PairformerModule(384, 128, 2, v2=True)
    assert list(m.state_dict().keys()) == list(sd.keys())
    m.load_state_dict(sd, strict=True)
    assert torch.equal(m.layers[1].tri_mul_in.p_in.weight, sd["layers.1.tri_mul_in.p_in.weight"])
    sd2 = synthetic.make_weights(2, seed=1, with_s=False)
    m2 = B200PairformerNoSeqModule(128, 2)
    assert list(m2.state_dict().keys()) == list(sd2.keys())
    m2.load_state_dict(sd2, strict=True)


def test_cpu_inputs_are_refused():
    m = B200PairformerModule(384, 128, 1)
    s, z = synthetic.make_inputs(8)
    with pytest.raises(RuntimeError, match="CUDA"):
        m(s, z, None, None)
