"""Other pair widths than the trunk's 128: the template stack (c_z = 64), the c_z = 256 / 8-head blocks of the sibling
models and the attention-free pair update block run on the un-fused fp32 kernels and must meet that tier's tolerance
against the CPU oracle (1e-4 relative L2 per block; call sites: tt_bio/boltz2.py:3749-3753, tt_bio/protenix.py:947,
tt_bio/esmfold2.py:129-154)."""
import pytest
import torch

from oracle import pairformer_oracle as orc
from tests.conftest import rel_l2
from tt_boltz_b200 import B200PairformerModule, B200PairformerNoSeqModule, B200PairUpdateBlock, _lib, synthetic

pytestmark = pytest.mark.gpu
TOL = 1e-4


def test_template_stack_width_64():
    n, blocks = 40, 2
    sd = synthetic.make_weights(blocks, affine_jitter=0.2, std=0.05, with_s=False, c_z=64)
    _, z = synthetic.make_inputs(n, c_z=64, seed=4, with_s=False)
    _, pm, _ = synthetic.chain_block_mask(n, 3, n_pad=3, seed=2, keep_inter_chain=False)
    mod = B200PairformerNoSeqModule(64, blocks, precision="auto")
    mod.load_state_dict(sd, strict=True)
    got = mod.cuda()(z.cuda(), pm.cuda())
    torch.cuda.synchronize()
    with torch.no_grad():
        _, want = orc.pairformer_stack(None, z[0], None, pm[0], sd, blocks)
    assert _lib.device_status() == 0
    assert rel_l2(got[0].cpu(), want) < TOL


def test_width_256_with_eight_triangle_heads_and_single_track():
    n = 24
    dims = dict(c_s=384, c_z=256, num_heads=16, tri_heads=8, tri_head_dim=32)
    sd = synthetic.make_weights(1, affine_jitter=0.2, std=0.04, **dims)
    s, z = synthetic.make_inputs(n, c_z=256, seed=5)
    m, pm = synthetic.tail_padding_mask(n, 3)
    mod = B200PairformerModule(384, 256, 1, pairwise_num_heads=8, precision="auto")
    mod.load_state_dict(sd, strict=True)
    s_o, z_o = mod.cuda()(s.cuda(), z.cuda(), m.cuda(), pm.cuda())
    torch.cuda.synchronize()
    with torch.no_grad():
        s_w, z_w = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, 1)
    assert _lib.device_status() == 0
    assert rel_l2(z_o[0].cpu(), z_w) < TOL
    assert rel_l2(s_o[0].cpu(), s_w) < TOL


def test_pair_update_block_width_256():
    n, c, hidden = 33, 256, 512
    blk = B200PairUpdateBlock(c, hidden)
    g = torch.Generator().manual_seed(3)
    sd = {}
    for k, v in blk.state_dict().items():
        if k.endswith("norm_in.weight") or k.endswith("norm_out.weight") or k.endswith("norm.weight"):
            sd[k] = 1 + 0.2 * torch.randn(v.shape, generator=g)
        elif k.endswith(".bias"):
            sd[k] = 0.2 * torch.randn(v.shape, generator=g)
        else:
            sd[k] = 0.04 * torch.randn(v.shape, generator=g)
    blk.load_state_dict(sd, strict=True)
    _, z = synthetic.make_inputs(n, c_z=c, seed=8, with_s=False)
    _, pm = synthetic.tail_padding_mask(n, 2)
    got = blk.cuda()(z.cuda(), pm.cuda())
    torch.cuda.synchronize()
    with torch.no_grad():
        zz = z[0]
        zz = zz + orc.tri_mul(zz, sd, "tri_mul_out", pm[0], False)
        zz = zz + orc.tri_mul(zz, sd, "tri_mul_in", pm[0], True)
        zz = zz + orc.transition(zz, sd, "transition_z")
    assert _lib.device_status() == 0
    assert rel_l2(got[0].cpu(), zz) < TOL


def test_esmfold2_block_from_the_reference_model_through_the_remap():
    """tests/golden/remaps/esmfold2_block_c64_n14.npz holds what the reference's vendored PyTorch ESMFold2
    PairUpdateBlock (tt_bio/_vendor/esmfold2_hf/modeling_esmfold2_common.py) returns for weights under ITS key names;
    the same checkpoint through remaps.esmfold2_pair_update_block and the GPU block must reproduce it."""
    from tests.test_remaps import load_esmfold2_case
    from tt_boltz_b200 import remaps
    theirs, z, mask, want = load_esmfold2_case("esmfold2_block_c64_n14")
    ours = remaps.esmfold2_pair_update_block(theirs)
    blk = B200PairUpdateBlock(z.shape[-1], ours["transition_z.fc1.weight"].shape[0])
    blk.load_state_dict(ours, strict=True)
    got = blk.cuda()(z.cuda(), mask.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(got[0].cpu(), want[0]) < TOL


@pytest.mark.parametrize("name", ["template_noseq2_c64_n20_chain", "layer_c256_h8_n12_general"])
def test_other_widths_against_the_reference_modules(golden_dir, name):
    """tests/golden/widths/*.npz: what the reference's own PairformerNoSeqModule(64, 2) (the template stack) and
    PairformerModule(384, 256, 1, pairwise_num_heads=8) return in fp32; the GPU modules must reproduce them."""
    from tests.test_oracle_golden import load_width_case
    g, sd, s, z, m, pm = load_width_case(golden_dir, name)
    c_z, heads, blocks = int(g["c_z"]), int(g["tri_heads"]), int(g["blocks"])
    if s is None:
        mod = B200PairformerNoSeqModule(c_z, blocks, pairwise_num_heads=heads, precision="auto")
        mod.load_state_dict(sd, strict=True)
        z_o = mod.cuda()(z.cuda(), pm.cuda())
    else:
        mod = B200PairformerModule(384, c_z, blocks, pairwise_num_heads=heads, precision="auto")
        mod.load_state_dict(sd, strict=True)
        s_o, z_o = mod.cuda()(s.cuda(), z.cuda(), m.cuda(), pm.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(z_o[0].cpu(), torch.from_numpy(g["z_out"])[0]) < TOL
    if s is not None:
        assert rel_l2(s_o[0].cpu(), torch.from_numpy(g["s_out"])[0]) < TOL
