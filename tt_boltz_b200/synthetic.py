"""Seeded synthetic weights, inputs and masks for the Pairformer path.

Everything is drawn on the CPU in fp32 from ``torch.Generator`` objects in a fixed order, so
the CPU oracle and the CUDA path see identical values.  Key names and shapes are the
reference's state-dict keys for one ``PairformerLayer`` (tt_bio/reference.py:825-863 and the
sub-modules it builds), prefixed ``layers.{i}.`` inside a stack (reference.py:943-956).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch


def layer_param_shapes(c_s: int = 384, c_z: int = 128, num_heads: int = 16, tri_heads: int = 4,
                       tri_head_dim: int = 32, with_s: bool = True) -> List[Tuple[str, Tuple[int, ...]]]:
    """(name, shape) for every parameter of one layer, in the reference's registration order."""
    d = c_z          # triangle-multiplication hidden width equals c_z (reference.py:401-407)
    hd = tri_heads * tri_head_dim
    out: List[Tuple[str, Tuple[int, ...]]] = []
    if with_s:
        out += [("pre_norm_s.weight", (c_s,)), ("pre_norm_s.bias", (c_s,)),
                ("attention.proj_q.weight", (c_s, c_s)), ("attention.proj_q.bias", (c_s,)),
                ("attention.proj_k.weight", (c_s, c_s)), ("attention.proj_v.weight", (c_s, c_s)),
                ("attention.proj_g.weight", (c_s, c_s)),
                ("attention.proj_z.0.weight", (c_z,)), ("attention.proj_z.0.bias", (c_z,)),
                ("attention.proj_z.1.weight", (num_heads, c_z)),
                ("attention.proj_o.weight", (c_s, c_s))]
    for name in ("tri_mul_out", "tri_mul_in"):
        out += [(f"{name}.norm_in.weight", (c_z,)), (f"{name}.norm_in.bias", (c_z,)),
                (f"{name}.p_in.weight", (2 * d, c_z)), (f"{name}.g_in.weight", (2 * d, c_z)),
                (f"{name}.norm_out.weight", (d,)), (f"{name}.norm_out.bias", (d,)),
                (f"{name}.p_out.weight", (c_z, d)), (f"{name}.g_out.weight", (c_z, c_z))]
    for name in ("tri_att_start", "tri_att_end"):
        out += [(f"{name}.layer_norm.weight", (c_z,)), (f"{name}.layer_norm.bias", (c_z,)),
                (f"{name}.linear.weight", (tri_heads, c_z)),
                (f"{name}.mha.linear_q.weight", (hd, c_z)), (f"{name}.mha.linear_k.weight", (hd, c_z)),
                (f"{name}.mha.linear_v.weight", (hd, c_z)), (f"{name}.mha.linear_o.weight", (c_z, hd)),
                (f"{name}.mha.linear_g.weight", (hd, c_z))]
    if with_s:
        out += [("transition_s.norm.weight", (c_s,)), ("transition_s.norm.bias", (c_s,)),
                ("transition_s.fc1.weight", (4 * c_s, c_s)), ("transition_s.fc2.weight", (4 * c_s, c_s)),
                ("transition_s.fc3.weight", (c_s, 4 * c_s))]
    out += [("transition_z.norm.weight", (c_z,)), ("transition_z.norm.bias", (c_z,)),
            ("transition_z.fc1.weight", (4 * c_z, c_z)), ("transition_z.fc2.weight", (4 * c_z, c_z)),
            ("transition_z.fc3.weight", (c_z, 4 * c_z))]
    return out


def make_weights(num_blocks: int, seed: int = 1, std: float = 0.02, affine_jitter: float = 0.0,
                 with_s: bool = True, bf16_round: bool = False, **dims) -> Dict[str, torch.Tensor]:
    """Flat state dict ``layers.{i}.<name>`` of random-init weights.

    Matrices and the one linear bias are N(0, std).  LayerNorm gains are 1 and offsets 0 unless
    ``affine_jitter`` > 0, in which case gain = 1 + jitter*N(0,1) and offset = jitter*N(0,1)
    (used by parity tests so that the affine terms are exercised).
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    sd: Dict[str, torch.Tensor] = {}
    for i in range(num_blocks):
        for name, shape in layer_param_shapes(with_s=with_s, **dims):
            if len(shape) == 2 or name.endswith("proj_q.bias"):
                t = torch.randn(shape, generator=g) * std
            elif name.endswith(".weight"):
                t = torch.ones(shape)
                if affine_jitter:
                    t = t + affine_jitter * torch.randn(shape, generator=g)
            else:
                t = torch.zeros(shape)
                if affine_jitter:
                    t = affine_jitter * torch.randn(shape, generator=g)
            if bf16_round:
                t = t.bfloat16().float()
            sd[f"layers.{i}.{name}"] = t
    return sd


def make_inputs(n: int, c_s: int = 384, c_z: int = 128, seed: int = 0, with_s: bool = True,
                bf16_round: bool = False, scale_s: float = 1.0, scale_z: float = 1.0
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """s [1,n,c_s] then z [1,n,n,c_z], both N(0,1) from one generator (s drawn first)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = torch.randn(1, n, c_s, generator=g) * scale_s if with_s else None
    z = torch.randn(1, n, n, c_z, generator=g) * scale_z
    if bf16_round:
        z = z.bfloat16().float()
        if s is not None:
            s = s.bfloat16().float()
    return s, z


def tail_padding_mask(n: int, n_pad: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token mask with the last ``n_pad`` tokens zero, and its outer-product pair mask."""
    m = torch.ones(1, n)
    if n_pad:
        m[:, n - n_pad:] = 0
    return m, m[:, :, None] * m[:, None, :]


def random_padding_mask(n: int, frac: float, seed: int = 3) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token mask with a random ``frac`` of tokens zero, and its outer-product pair mask."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = (torch.rand(1, n, generator=g) >= frac).float()
    return m, m[:, :, None] * m[:, None, :]


def chain_block_mask(n: int, n_chains: int = 3, n_pad: int = 0, seed: int = 2,
                     keep_inter_chain: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Random chain lengths summing to n; pair mask either outer(token mask) or block-diagonal."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    cuts = torch.sort(torch.randperm(n - 1, generator=g)[: n_chains - 1] + 1).values.tolist()
    bounds = [0] + cuts + [n]
    chain_id = torch.zeros(n, dtype=torch.long)
    for c in range(n_chains):
        chain_id[bounds[c]:bounds[c + 1]] = c
    m, pm = tail_padding_mask(n, n_pad)
    if not keep_inter_chain:
        pm = pm * (chain_id[:, None] == chain_id[None, :]).float()[None]
    return m, pm, chain_id


def sampled_fixture_errors(fixture, blocks: int, s_out: torch.Tensor, z_out: torch.Tensor) -> Tuple[float, float]:
    """rel-L2 of (s_out [N, c_s], z_out [N, N, c_z]) against a sampled full-size fixture (an ``np.load`` of a file
    written by tests/golden/make_sampled_trunk.py) after ``blocks`` blocks: z over the fixture's sampled positions,
    s over the whole tensor; positions of masked tokens (the fixture's ``mask``) are left out, the reference does
    not define them.  Works on any device; returns (rel_l2_z, rel_l2_s)."""
    n, c = z_out.shape[0], z_out.shape[-1]
    idx = torch.from_numpy(fixture["index"]).to(z_out.device)
    z_ref = torch.from_numpy(fixture[f"z_samples_{blocks}"]).to(z_out.device).double()
    s_ref = torch.from_numpy(fixture[f"s_{blocks}"]).to(s_out.device).double()
    z_got = z_out.reshape(-1)[idx].double()
    s_got = s_out.double()
    if "mask" in getattr(fixture, "files", fixture):
        m = torch.from_numpy(fixture["mask"]).to(z_out.device) != 0
        if not bool(m.all()):
            ok = m[idx // (n * c)] & m[(idx // c) % n]
            z_got, z_ref = z_got[ok], z_ref[ok]
            s_got, s_ref = s_got[m.to(s_out.device)], s_ref[m.to(s_out.device)]
    rz = float((z_got - z_ref).norm() / z_ref.norm())
    rs = float((s_got - s_ref).norm() / s_ref.norm())
    return rz, rs


def make_opm_weights(seed: int = 11, c_in: int = 64, c_hidden: int = 32, c_out: int = 128, std: float = 0.05,
                     affine_jitter: float = 0.2) -> Dict[str, torch.Tensor]:
    """State dict of the outer-product mean with the reference's key names (tt_bio/reference.py:590-596); every
    parameter random so that nothing the upstream zero-initialises (proj_o) hides an error."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return {
        "norm.weight": 1 + affine_jitter * torch.randn(c_in, generator=g),
        "norm.bias": affine_jitter * torch.randn(c_in, generator=g),
        "proj_a.weight": torch.randn(c_hidden, c_in, generator=g) * std * 4,
        "proj_b.weight": torch.randn(c_hidden, c_in, generator=g) * std * 4,
        "proj_o.weight": torch.randn(c_out, c_hidden * c_hidden, generator=g) * std,
        "proj_o.bias": torch.randn(c_out, generator=g) * std,
    }


def make_msa_inputs(s: int, n: int, c_in: int = 64, drop: float = 0.0, seed: int = 5) -> Tuple[torch.Tensor, torch.Tensor]:
    """MSA activations m [s, n, c_in] ~ N(0.3, 1) and a mask [s, n] of ones with a share `drop` of zeros (the first
    sequence, the query, is never masked)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.randn(s, n, c_in, generator=g) + 0.3
    mask = (torch.rand(s, n, generator=g) >= drop).float()
    mask[0] = 1.0
    return m, mask


def make_msa_layer_weights(seed: int = 21, std: float = 0.05, affine_jitter: float = 0.2) -> Dict[str, torch.Tensor]:
    """State dict of one MSA layer with the reference's key names (tt_bio/reference.py:1336-1358): transition and
    pair-weighted averaging on the 64-channel MSA activations, outer-product mean, and a pair-only Pairformer block."""
    g = torch.Generator(device="cpu").manual_seed(seed)

    def mat(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * std * scale

    def gain(c):
        return 1 + affine_jitter * torch.randn(c, generator=g)

    def offset(c):
        return affine_jitter * torch.randn(c, generator=g)

    sd = {
        "msa_transition.norm.weight": gain(64), "msa_transition.norm.bias": offset(64),
        "msa_transition.fc1.weight": mat(256, 64, scale=2), "msa_transition.fc2.weight": mat(256, 64, scale=2),
        "msa_transition.fc3.weight": mat(64, 256, scale=2),
        "pair_weighted_averaging.norm_m.weight": gain(64), "pair_weighted_averaging.norm_m.bias": offset(64),
        "pair_weighted_averaging.norm_z.weight": gain(128), "pair_weighted_averaging.norm_z.bias": offset(128),
        "pair_weighted_averaging.proj_m.weight": mat(256, 64, scale=2), "pair_weighted_averaging.proj_g.weight": mat(256, 64, scale=2),
        "pair_weighted_averaging.proj_z.weight": mat(8, 128, scale=4), "pair_weighted_averaging.proj_o.weight": mat(64, 256, scale=2),
    }
    for k, v in make_opm_weights(seed=seed + 1).items():
        sd["outer_product_mean." + k] = v
    for k, v in make_weights(1, seed=seed + 2, std=std, affine_jitter=affine_jitter, with_s=False).items():
        sd["pairformer_layer." + k[len("layers.0."):]] = v
    return sd


def make_msa_module_weights(blocks: int = 2, seed: int = 31) -> Dict[str, torch.Tensor]:
    """State dict of the MSA module with the reference's key names (tt_bio/reference.py:1187-1201): the two input
    projections and ``layers.{i}.*`` of ``make_msa_layer_weights``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    sd = {"s_proj.weight": torch.randn(64, 384, generator=g) * 0.05, "msa_proj.weight": torch.randn(64, 36, generator=g) * 0.3}
    for i in range(blocks):
        for k, v in make_msa_layer_weights(seed=seed + 10 * (i + 1)).items():
            sd[f"layers.{i}.{k}"] = v
    return sd


def make_msa_features(s: int, n: int, n_pad: int = 0, drop: float = 0.2, seed: int = 13) -> Dict[str, torch.Tensor]:
    """The MSA entries of the feature dict the MSA module reads (tt_bio/reference.py:1252-1259), batch 1."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    mask = (torch.rand(1, s, n, generator=g) >= drop).float()
    mask[:, 0] = 1.0
    pad = torch.ones(1, n)
    if n_pad:
        pad[:, n - n_pad:] = 0
    return {
        "msa": torch.randint(0, 33, (1, s, n), generator=g),
        "has_deletion": (torch.rand(1, s, n, generator=g) < 0.1).float(),
        "deletion_value": torch.rand(1, s, n, generator=g),
        "msa_paired": (torch.rand(1, s, n, generator=g) < 0.5).float(),
        "msa_mask": mask,
        "token_pad_mask": pad,
    }
