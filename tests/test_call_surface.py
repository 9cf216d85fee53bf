"""The module classes must be constructible and loadable the way every call site of the reference does it.

Two constructor conventions exist in the reference: the CPU modules' (tt_bio/reference.py:921-934, 1096-1108)
and the device backend's (tt_bio/tenstorrent.py:2194-2204), which is what the template (boltz2.py:3751),
confidence (:4503), affinity (:4689) and trunk (:5016) call sites build when the backend is selected.
No GPU is needed: nothing here runs a kernel.
"""
import inspect

import pytest
import torch

from tt_boltz_b200 import (B200MSALayer, B200MSAModule, B200MSATransition, B200OuterProductMean, B200PairWeightedAveraging, B200PairformerLayer, B200PairformerModule, B200PairformerNoSeqLayer,
                           B200PairformerNoSeqModule, B200RecyclingTrunk, synthetic)
from tt_boltz_b200 import B200DistogramModule


def _params(fn):
    return list(inspect.signature(fn).parameters)


def test_forward_signatures_match_the_reference():
    # tt_bio/reference.py:958-965 and tt_bio/tenstorrent.py:2227-2234
    assert _params(B200PairformerModule.forward) == ["self", "s", "z", "mask", "pair_mask", "use_kernels"]
    # tt_bio/reference.py:865-875
    assert _params(B200PairformerLayer.forward)[:7] == ["self", "s", "z", "mask", "pair_mask", "chunk_size_tri_attn", "use_kernels"]
    # tt_bio/reference.py:1034-1042
    assert _params(B200PairformerNoSeqLayer.forward) == ["self", "z", "pair_mask", "chunk_size_tri_attn", "use_kernels",
                                                         "use_cuequiv_mul", "use_cuequiv_attn"]
    # tt_bio/reference.py:1109-1114
    assert _params(B200PairformerNoSeqModule.forward) == ["self", "z", "pair_mask", "use_kernels"]


@pytest.mark.parametrize("args, with_s, blocks", [
    ((64, 32, 4, 24, 16, True), True, 64),          # trunk, boltz2.py:5016
    ((8, 32, 4, 24, 16, True), True, 8),            # confidence, boltz2.py:4503
    ((2, 32, 4, None, None, False), False, 2),      # templates, boltz2.py:3751
])
def test_backend_style_constructor(args, with_s, blocks):
    mod = B200PairformerModule(*args)
    assert mod.transform_s is with_s and len(mod.layers) == blocks
    keys = set(mod.state_dict().keys())
    assert keys == set(synthetic.make_weights(blocks, with_s=with_s).keys())
    assert ("layers.0.pre_norm_s.weight" in keys) is with_s


def test_backend_style_keywords_and_affinity_flag():
    mod = B200PairformerModule(n_blocks=4, tri_att_head_dim=32, tri_att_n_heads=4, att_head_dim=None,
                               att_n_heads=None, transform_s=False, affinity=True)
    assert mod.affinity and not mod.transform_s and len(mod.layers) == 4


def test_cpu_module_style_constructor_still_works():
    mod = B200PairformerModule(384, 128, 3, num_heads=16, dropout=0.25, pairwise_head_width=32,
                               pairwise_num_heads=4, post_layer_norm=False, activation_checkpointing=False, v2=True)
    assert mod.transform_s and len(mod.layers) == 3
    mod.load_state_dict(synthetic.make_weights(3), strict=True)
    with pytest.raises(TypeError):
        B200PairformerModule(384, 128)


@pytest.mark.parametrize("with_s", [True, False])
def test_load_state_dict_with_the_backend_key_convention(with_s):
    """The backend reads the triangle-attention projections with the ``mha.`` level stripped
    (tt_bio/tenstorrent.py:973, 981); both spellings must load, strictly, to the same parameters."""
    sd = synthetic.make_weights(2, with_s=with_s)
    stripped = {k.replace(".mha.", "."): v for k, v in sd.items()}
    assert any(k not in sd for k in stripped)
    a = B200PairformerModule(2, 32, 4, 24 if with_s else None, 16 if with_s else None, with_s)
    b = B200PairformerModule(2, 32, 4, 24 if with_s else None, 16 if with_s else None, with_s)
    a.load_state_dict(sd, strict=True)
    b.load_state_dict(stripped, strict=True)
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)
    layer = B200PairformerNoSeqLayer(128)
    one = {k[len("layers.0."):].replace("mha.", ""): v for k, v in synthetic.make_weights(1, with_s=False).items()}
    layer.load_state_dict(one, strict=True)


def test_no_cpu_path_on_any_surface():
    z = torch.zeros(1, 8, 8, 128)
    pm = torch.ones(1, 8, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        B200PairformerModule(1, 32, 4, None, None, False)(None, z, None, pm)
    with pytest.raises(RuntimeError, match="CUDA"):
        B200PairformerNoSeqLayer(128)(z, pm)
    with pytest.raises(RuntimeError, match="single track"):
        B200PairformerModule(1, 32, 4, 24, 16, True)(None, z.cuda() if torch.cuda.is_available() else z, None, pm)


def test_recycling_trunk_carries_the_reference_key_names():
    """tt_bio/boltz2.py:4961-4966 names the recycle parameters; `pairformer_module.` prefixes the stack (:5015)."""
    trunk = B200RecyclingTrunk(B200PairformerModule(64, 32, 4, 24, 16, True))
    keys = set(trunk.state_dict().keys())
    for k in ("s_norm.weight", "s_norm.bias", "z_norm.weight", "z_norm.bias", "s_recycle.weight", "z_recycle.weight",
              "pairformer_module.layers.63.transition_z.fc3.weight"):
        assert k in keys, k
    assert _params(B200RecyclingTrunk.forward) == ["self", "s_init", "z_init", "mask", "pair_mask", "recycling_steps", "pair_update"]
    with pytest.raises(RuntimeError, match="CUDA"):
        trunk(torch.zeros(1, 8, 384), torch.zeros(1, 8, 8, 128))


def test_outer_product_mean_surface():
    """tt_bio/reference.py:574-597: constructor (c_in, c_hidden, c_out), forward(m, mask, chunk_size), six parameters."""
    mod = B200OuterProductMean(64, 32, 128)
    assert _params(B200OuterProductMean.forward) == ["self", "m", "mask", "chunk_size"]
    assert set(mod.state_dict().keys()) == set(synthetic.make_opm_weights().keys())
    mod.load_state_dict(synthetic.make_opm_weights(), strict=True)
    with pytest.raises(ValueError):
        B200OuterProductMean(64, 16, 128)
    m, mask = synthetic.make_msa_inputs(4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(m[None], mask[None])


def test_msa_layer_surface():
    """tt_bio/reference.py:1314-1376: constructor (msa_s, token_z, msa_dropout, z_dropout, head width, heads), the four
    sub-modules by name, forward(z, m, token_mask, msa_mask, five chunk arguments, use_kernels) -> (z, m)."""
    layer = B200MSALayer(64, 128, 0.0, 0.0)
    assert set(layer.state_dict().keys()) == set(synthetic.make_msa_layer_weights().keys())
    layer.load_state_dict(synthetic.make_msa_layer_weights(), strict=True)
    assert _params(B200MSALayer.forward) == ["self", "z", "m", "token_mask", "msa_mask", "chunk_heads_pwa", "chunk_size_transition_z",
                                             "chunk_size_transition_msa", "chunk_size_outer_product", "chunk_size_tri_attn", "use_kernels"]
    # reference.py:727-729 and boltz2.py:1227
    assert _params(B200PairWeightedAveraging.forward) == ["self", "m", "z", "mask", "chunk_heads"]
    assert _params(B200MSATransition.forward) == ["self", "x", "chunk_size"]
    z = torch.zeros(1, 8, 8, 128)
    m, msa_mask = synthetic.make_msa_inputs(4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(z, m[None], torch.ones(1, 8, 8), msa_mask[None])
    with pytest.raises(RuntimeError, match="CUDA"):
        layer.pair_weighted_averaging(m[None], z, torch.ones(1, 8, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        layer.msa_transition(m[None])


def test_msa_module_surface():
    """tt_bio/reference.py:1153-1201, 1203-1209: constructor keywords, parameters, forward(z, emb, feats, use_kernels)."""
    mod = B200MSAModule(msa_s=64, token_z=128, token_s=384, msa_blocks=4, msa_dropout=0.15, z_dropout=0.25,
                        pairwise_head_width=32, pairwise_num_heads=4, activation_checkpointing=False,
                        use_paired_feature=True, subsample_msa=False, num_subsampled_msa=1024)
    assert set(mod.state_dict().keys()) == set(synthetic.make_msa_module_weights(4).keys())
    assert _params(B200MSAModule.forward) == ["self", "z", "emb", "feats", "use_kernels"]
    feats = synthetic.make_msa_features(4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(torch.zeros(1, 8, 8, 128), torch.zeros(1, 8, 384), feats)


def test_distogram_head_surface_and_fixture():
    """tests/golden/heads/distogram_n12.npz holds the reference's DistogramModule (tt_bio/boltz2.py:2334-2368): its
    state dict loads strictly into ours, the stored output is Linear(z + z^T) of the stored input, and there is no CPU
    path."""
    import os
    import numpy as np
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "heads", "distogram_n12.npz"))
    w = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("w::")}
    head = B200DistogramModule(128, 64)
    head.load_state_dict(w, strict=True)
    assert _params(B200DistogramModule.forward) == ["self", "z"]
    z, out = torch.from_numpy(g["z"]), torch.from_numpy(g["out"])
    want = (z + z.transpose(1, 2)) @ w["distogram.weight"].T + w["distogram.bias"]
    assert out.shape == (1, 12, 12, 1, 64) and torch.allclose(out[:, :, :, 0], want, atol=1e-5)
    with pytest.raises(RuntimeError, match="CUDA"):
        head(z)
