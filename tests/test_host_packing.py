"""Host logic: weight packing and the module's state-dict surface, checked on the CPU.

The kernels cannot run here, so each packing layout is validated by a small torch model of what
the kernel does with the packed buffers (LayerNorm with the affine, multiply by the packed bf16
rows, combine the values the layout puts side by side) against the oracle.
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


def ln_affine(z, gamma, beta):
    return xhat(z) * gamma + beta


@pytest.mark.parametrize("incoming", [False, True])
def test_trimul_packing_model(setup, incoming):
    """What the producer and the epilogue kernels do with their packed weights: halved p / g rows so that
    p * sigmoid(g) = p' + p' * tanh(g'), and the epilogue's LayerNorm over channels applied AFTER the GEMM
    (p = rstd * (acc - mean * wsum) + wb)."""
    sd, z, pm = setup
    pre = "tri_mul_in" if incoming else "tri_mul_out"
    pk = weights.pack_trimul(sd, pre + ".", "cpu")
    assert pk["w_pg_tc"].shape == (512, 128)
    x = ln_affine(z, pk["ln_in_gamma"], pk["ln_in_beta"])
    y = x @ pk["w_pg_tc"].float().T                                  # [N,N,512] = 0.5 * [p_a | g_a | p_b | g_b]
    gated = lambda pp, gg: (pp + pp * torch.tanh(gg)) * pm[..., None]
    a, b = gated(y[..., 0:128], y[..., 128:256]), gated(y[..., 256:384], y[..., 384:512])
    t = torch.einsum("kic,kjc->ijc", a, b) if incoming else torch.einsum("ikc,jkc->ijc", a, b)
    acc = t @ pk["w_pout_tc"].float().T                              # raw x against 0.5 * W_pout * gamma_out
    mean = t.mean(-1, keepdim=True)
    rstd = torch.rsqrt(((t - mean) ** 2).mean(-1, keepdim=True) + 1e-5)
    pp = rstd * (acc - mean * pk["wsum_tc"]) + pk["wb_tc"]
    gg = x @ pk["w_gout_tc"].float().T
    upd = pp + pp * torch.tanh(gg)
    ref = orc.tri_mul(z, sd, pre, pm, incoming)
    assert rel_l2(upd, ref) < 1e-2


@pytest.mark.parametrize("ending", [False, True])
def test_triatt_packing_model(setup, ending):
    sd, z, pm = setup
    pre = "tri_att_end" if ending else "tri_att_start"
    pk = weights.pack_triatt(sd, pre + ".", "cpu")
    assert pk["w_qkgv_tc"].shape == (512, 128) and pk["w_bias_f32"].shape == (4, 128)
    x = ln_affine(z, pk["ln_gamma"], pk["ln_beta"])
    y = x @ pk["w_qkgv_tc"].float().T                                # [N,N,512] in z layout (r, c): q | k | 0.5 g | v
    bias = x @ pk["w_bias_f32"].T                                    # [r, c, h], log2 domain
    if ending:          # line = column: (line, pos) = (c, r)
        y, bias = y.transpose(0, 1), bias.transpose(0, 1)
        mask = pm.T
    else:
        mask = pm
    q, k = (y[..., i * 128:(i + 1) * 128].reshape(N, N, 4, 32) for i in range(2))
    v = y[..., 384:512].reshape(N, N, 4, 32)
    gate = 0.5 + 0.5 * torch.tanh(y[..., 256:384])
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
    assert pk["w12_tc"].shape == (8, 128, 128) and pk["w3"].shape == (8, 128, 64)
    x = ln_affine(z, pk["ln_gamma"], pk["ln_beta"])
    out = torch.zeros(N, N, 128)
    for c in range(8):
        y = x @ pk["w12_tc"][c].float().T                           # [N,N,128] = 0.5 * fc1 chunk | fc2 chunk
        a, f2 = y[..., :64], y[..., 64:]
        h = (a + a * torch.tanh(a)) * f2                             # silu(f1) * f2 with a = f1 / 2
        out += h @ pk["w3"][c].float().T
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
