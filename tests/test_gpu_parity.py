"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the golden
fixtures made from the reference's own CPU modules.

Tolerances (rel-L2 = ||x - ref|| / ||ref||):
  fp32 tier  : <= 1e-4 on z and s per layer
  bf16 tier  : <= 2e-2 (sub-operation updates and stacked layers)
Mask handling: values stored at masked-out tokens must not change the valid region at all.
"""
import ctypes as C
import glob
import os

import numpy as np
import pytest
import torch

from oracle import pairformer_oracle as orc
from tests.conftest import rel_l2
from tt_boltz_b200 import B200PairformerLayer, B200PairformerModule, B200PairformerNoSeqModule, synthetic

pytestmark = pytest.mark.gpu
GOLDEN = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def strip(sd, i=0):
    pre = f"layers.{i}."
    return {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}


def run_module(sd, blocks, s, z, m, pm, dev, precision, with_s=True, **attrs):
    if with_s:
        mod = B200PairformerModule(384, 128, blocks, v2=True, precision=precision)
    else:
        mod = B200PairformerNoSeqModule(128, blocks, precision=precision)
    mod.load_state_dict(sd, strict=True)
    for layer in mod.layers:
        for k, v in attrs.items():
            setattr(layer, k, v)
    if with_s:
        so, zo = mod(s.to(dev), z.to(dev), m.to(dev), pm.to(dev))
        return so.cpu(), zo.cpu()
    return None, mod(z.to(dev), pm.to(dev)).cpu()


# ---------------------------------------------------------------------------------------------
# golden fixtures (outputs of the reference's CPU modules)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("precision,tol", [("fp32", 1e-4), ("bf16", 2e-2)])
@pytest.mark.parametrize("name", GOLDEN)
def test_golden_fixture(golden_dir, dev, name, precision, tol):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    n, nb, with_s = int(g["n"]), int(g["blocks"]), bool(g["with_s"])
    sd = synthetic.make_weights(nb, seed=1, std=float(g["std"]), affine_jitter=float(g["jitter"]), with_s=with_s)
    s, z = synthetic.make_inputs(n, seed=0, with_s=with_s)
    m, pm = torch.from_numpy(g["mask"]), torch.from_numpy(g["pair_mask"])
    so, zo = run_module(sd, nb, s, z, m, pm, dev, precision, with_s)
    valid = m[0].bool()
    zr = torch.from_numpy(g["z_out"])
    assert torch.isfinite(zo).all()
    assert rel_l2(zo[0][valid][:, valid], zr[0][valid][:, valid]) < tol
    if with_s:
        sr = torch.from_numpy(g["s_out"])
        assert rel_l2(so[0][valid], sr[0][valid]) < tol


# ---------------------------------------------------------------------------------------------
# configuration 1 of the benchmark: one layer, fp32, N = 128, all-ones masks, N(0, 0.02) weights
# ---------------------------------------------------------------------------------------------
def test_cfg1_layer_fp32_n128(dev):
    n = 128
    sd = synthetic.make_weights(1, seed=1)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 0)
    so, zo = run_module(sd, 1, s, z, m, pm, dev, "fp32")
    sr, zr = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, 1)
    assert rel_l2(zo[0], zr) < 1e-4
    assert rel_l2(so[0], sr) < 1e-4
    # the bf16 tier on the same input
    so, zo = run_module(sd, 1, s, z, m, pm, dev, "bf16")
    assert rel_l2(zo[0], zr) < 2e-2 and rel_l2(so[0], sr) < 2e-2


# ---------------------------------------------------------------------------------------------
# sub-operations, bf16 tier, ragged sizes and general 2-D masks (update compared on its own)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [37, 100, 128, 200])
def test_sub_operations_bf16(dev, n):
    from tt_boltz_b200 import ops, weights
    sd = strip(synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3))
    _, z = synthetic.make_inputs(n, seed=4, with_s=False)
    g = torch.Generator().manual_seed(9)
    tm = torch.ones(n)
    tm[n - max(1, n // 10):] = 0
    pm = (torch.rand(n, n, generator=g) > 0.15).float() * tm[:, None] * tm[None, :]
    pm_u8 = (pm != 0).to(torch.uint8).to(dev)
    ws = ops.Workspace(n, dev)
    v = tm.bool()
    cases = [
        ("tri_mul_out", lambda zz: ops.tri_mul_bf16(zz, pm_u8, weights.pack_trimul(sd, "tri_mul_out.", dev), ws, False),
         lambda zc: orc.tri_mul(zc, sd, "tri_mul_out", pm, False)),
        ("tri_mul_in", lambda zz: ops.tri_mul_bf16(zz, pm_u8, weights.pack_trimul(sd, "tri_mul_in.", dev), ws, True),
         lambda zc: orc.tri_mul(zc, sd, "tri_mul_in", pm, True)),
        ("tri_att_start", lambda zz: ops.tri_att_bf16(zz, ops.PairMasks(pm_u8), weights.pack_triatt(sd, "tri_att_start.", dev), ws, False),
         lambda zc: orc.tri_att(zc, sd, "tri_att_start", pm, False)),
        ("tri_att_end", lambda zz: ops.tri_att_bf16(zz, ops.PairMasks(pm_u8), weights.pack_triatt(sd, "tri_att_end.", dev), ws, True),
         lambda zc: orc.tri_att(zc, sd, "tri_att_end", pm, True)),
        ("transition_z", lambda zz: ops.transition_z_bf16(zz, weights.pack_transition_z(sd, "transition_z.", dev)),
         lambda zc: orc.transition(zc, sd, "transition_z")),
    ]
    for name, run, ref in cases:
        zd = z[0].to(dev).clone()
        run(zd)
        torch.cuda.synchronize()
        upd = (zd.cpu() - z[0])
        want = ref(z[0])
        assert torch.isfinite(upd).all(), name
        assert rel_l2(upd[v][:, v], want[v][:, v]) < 2e-2, name


def test_contraction_tcgen05_matches_einsum(dev):
    from tt_boltz_b200._lib import Planes, call, ptr, stream
    from tt_boltz_b200 import _lib
    for n in (24, 100, 128, 264, 512):
        pitch = (n + 7) // 8 * 8
        ps = n * pitch
        g = torch.Generator().manual_seed(n)
        a = torch.randn(128, n, pitch, generator=g).bfloat16()
        b = torch.randn(128, n, pitch, generator=g).bfloat16()
        ad, bd = a.to(dev), b.to(dev)
        x = torch.zeros(128, n, pitch, dtype=torch.bfloat16, device=dev)
        pa = Planes(ptr(ad), ps, 0, pitch, n, n, 1, 0)
        pb = Planes(ptr(bd), ps, 0, pitch, n, n, 1, 0)
        call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), ps, pitch, 0, 0, 128, 0, stream())
        assert _lib.device_status() == 0
        ref = torch.einsum("dik,djk->dij", a[:, :, :n].float(), b[:, :, :n].float())
        assert rel_l2(x[:, :, :n].float().cpu(), ref) < 4e-3, n       # bf16 rounding of the stored result


@pytest.mark.parametrize("seg_is_k", [0, 1])
def test_contraction_segmented_operands_and_grouped_output(dev, seg_is_k):
    """The operand / result layouts of the channel-parallel sharded triangle multiplication: both operands split in
    P segments (blocks of rows, or blocks of the contraction index), the result written in P groups of output rows."""
    from tt_boltz_b200._lib import Planes, call, ptr, stream
    from tt_boltz_b200 import _lib
    world, cl, n = 2, 16, 256
    nr = n // world
    g = torch.Generator().manual_seed(31 + seg_is_k)
    a = torch.randn(cl, n, n, generator=g).bfloat16()          # [c][i][k]
    b = torch.randn(cl, n, n, generator=g).bfloat16()          # [c][j][k]
    if seg_is_k:    # segment s holds k in [s*nr, (s+1)*nr): [s][c][row][k local]
        a_seg = a.view(cl, n, world, nr).permute(2, 0, 1, 3).contiguous()
        b_seg = b.view(cl, n, world, nr).permute(2, 0, 1, 3).contiguous()
        rows, cols = n, nr
    else:           # segment s holds rows [s*nr, (s+1)*nr): [s][c][row local][k]
        a_seg = a.view(cl, world, nr, n).permute(1, 0, 2, 3).contiguous()
        b_seg = b.view(cl, world, nr, n).permute(1, 0, 2, 3).contiguous()
        rows, cols = nr, n
    ad, bd = a_seg.to(dev), b_seg.to(dev)
    ref = torch.einsum("cik,cjk->cij", a.float(), b.float())
    x = torch.zeros(world, cl, nr, n, dtype=torch.bfloat16, device=dev)        # [group = i / nr][c][i local][j]
    pa = Planes(ptr(ad), rows * cols, cl * rows * cols, cols, rows, cols, world, seg_is_k)
    pb = Planes(ptr(bd), rows * cols, cl * rows * cols, cols, rows, cols, world, seg_is_k)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), nr * n, n, nr, cl * nr * n, cl, 0, stream())
    assert _lib.device_status() == 0
    assert rel_l2(x.permute(1, 0, 2, 3).reshape(cl, n, n).float().cpu(), ref) < 4e-3


def test_fused_tier_matches_the_fp32_tier(dev):
    """One layer on the fused tcgen05 kernels against the same layer on the un-fused fp32 SIMT kernels: two
    independent implementations inside the library (besides the comparisons with the CPU oracle)."""
    n = 136
    sd = synthetic.make_weights(1, seed=1, std=0.05, affine_jitter=0.3)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 11)
    _, z_tc = run_module(sd, 1, s, z, m, pm, dev, "bf16")
    _, z_x = run_module(sd, 1, s, z, m, pm, dev, "fp32")
    v = n - 11
    assert rel_l2((z_tc - z)[0, :v, :v], (z_x - z)[0, :v, :v]) < 8e-3


@pytest.mark.parametrize("n", [50, 128, 200, 330])
def test_attention_core_against_fp32_tier_with_general_masks(dev, n):
    """Triangle attention (starting and ending node) on the tcgen05 path against the fp32 tier's un-fused kernels,
    with a random 2-D mask (most key tiles hold masked keys: the per-tile mask path) and one fully masked line."""
    from tt_boltz_b200 import _lib, ops, weights
    sd = strip(synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3))
    _, z = synthetic.make_inputs(n, seed=4, with_s=False)
    g = torch.Generator().manual_seed(9)
    pm = (torch.rand(n, n, generator=g) > 0.15).to(torch.uint8)
    pm[3, :] = 0                       # one fully masked line
    masks = ops.PairMasks(pm.to(dev))
    ws = ops.Workspace(n, dev)
    for ending in (False, True):
        pre = "tri_att_end." if ending else "tri_att_start."
        zd = z[0].to(dev).clone()
        ops.tri_att_bf16(zd, masks, weights.pack_triatt(sd, pre, dev), ws, ending)
        assert _lib.device_status() == 0
        zf = z[0].to(dev).clone()
        ops.tri_att_f32(zf, masks.pm, weights.to_device_f32(sd, pre, dev), ending)
        upd, ref = zd.cpu() - z[0], zf.cpu() - z[0]
        assert torch.isfinite(upd).all()
        assert rel_l2(upd, ref) < 7e-3, (n, ending)


@pytest.mark.parametrize("n", [72, 200])
def test_attention_with_bf16_input_and_stored_update(dev, n):
    """The forms the sharded ending node uses: the producer reading the pair tensor in bf16, the epilogue storing
    the update in bf16 instead of adding it.  Against the fp32-input / in-place forms on the same data."""
    from tt_boltz_b200 import _lib, ops, weights
    from tt_boltz_b200._lib import call, ptr, stream
    sd = strip(synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3))
    _, z = synthetic.make_inputs(n, seed=4, with_s=False)
    g = torch.Generator().manual_seed(9)
    pm = (torch.rand(n, n, generator=g) > 0.1).to(torch.uint8)
    masks = ops.PairMasks(pm.to(dev))
    ws = ops.Workspace(n, dev)
    for ending in (False, True):
        w = weights.pack_triatt(sd, "tri_att_end." if ending else "tri_att_start.", dev)
        z_ref = z[0].to(dev).clone()
        ops.tri_att_bf16(z_ref, masks, w, ws, ending)
        ref = z_ref.cpu() - z[0]
        # bf16 input, stored update
        z16 = z[0].to(dev).to(torch.bfloat16).contiguous()
        q, k, v, gg, o = ws.buf
        call("b200pf_triatt_producer_bf16z", ptr(z16), *ops.triatt_producer_weights(w), ptr(q), ptr(k), ptr(v), ptr(gg),
             ptr(ws.tri_bias), ws.pitch, 4 * ws.pitch, ws.pitch, n, n, int(ending), stream())
        o_ls, o_ps = (128, n * 128) if ending else (n * 128, 128)
        call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), ws.pitch, ptr(ws.tri_bias), ws.pitch, 4 * ws.pitch,
             ptr(masks.cols if ending else masks.rows), masks.pitch, ptr(o), o_ls, o_ps, n, n, stream())
        upd = torch.full((n * n * 128,), float("nan"), dtype=torch.bfloat16, device=dev)
        call("b200pf_triatt_epilogue_update", ptr(upd), ptr(o), ptr(gg), ptr(w["w_o"]), n * n, stream())
        assert _lib.device_status() == 0
        got = upd.float().cpu().view(n, n, 128)
        assert torch.isfinite(got).all()
        assert rel_l2(got, ref) < 8e-3, (n, ending)      # z rounded to bf16 before the LayerNorm, update rounded to bf16


# ---------------------------------------------------------------------------------------------
# masks: what is stored at masked-out tokens must not reach the valid region (bit-exact)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_padding_is_isolated_exactly(dev, precision):
    n, npad = 72, 9
    sd = synthetic.make_weights(1, seed=1, std=0.05, affine_jitter=0.2)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, npad)
    g = torch.Generator().manual_seed(11)
    z2, s2 = z.clone(), s.clone()
    z2[0, n - npad:] = 30 * torch.randn(npad, n, 128, generator=g)
    z2[0, :, n - npad:] = 30 * torch.randn(n, npad, 128, generator=g)
    s2[0, n - npad:] = 30 * torch.randn(npad, 384, generator=g)
    sa, za = run_module(sd, 1, s, z, m, pm, dev, precision)
    sb, zb = run_module(sd, 1, s2, z2, m, pm, dev, precision)
    v = n - npad
    assert torch.equal(za[0, :v, :v], zb[0, :v, :v])
    assert torch.equal(sa[0, :v], sb[0, :v])
    assert torch.isfinite(zb).all() and torch.isfinite(sb).all()


def test_full_size_properties_n1024(dev):
    """At the benchmark's token count the oracle takes minutes per block, so two size-independent properties stand in:
    (1) what is stored at padded tokens never reaches the valid region (bit-exact), (2) the trunk commutes with a
    permutation of the tokens (up to bf16 rounding: the permutation changes tile membership and summation order)."""
    n, npad, nb = 1024, 24, 2
    sd = synthetic.make_weights(nb, seed=3)
    s, z = synthetic.make_inputs(n, seed=5)
    m, pm = synthetic.tail_padding_mask(n, npad)
    g = torch.Generator().manual_seed(13)
    v = n - npad
    sa, za = run_module(sd, nb, s, z, m, pm, dev, "bf16")
    assert torch.isfinite(za).all() and torch.isfinite(sa).all()
    # (1) garbage in the padding
    z2, s2 = z.clone(), s.clone()
    z2[0, v:] = 30 * torch.randn(npad, n, 128, generator=g)
    z2[0, :, v:] = 30 * torch.randn(n, npad, 128, generator=g)
    s2[0, v:] = 30 * torch.randn(npad, 384, generator=g)
    sb, zb = run_module(sd, nb, s2, z2, m, pm, dev, "bf16")
    assert torch.equal(za[0, :v, :v], zb[0, :v, :v])
    assert torch.equal(sa[0, :v], sb[0, :v])
    del z2, s2, sb, zb
    # (2) permutation of the tokens
    perm = torch.randperm(n, generator=g)
    sp, zp = run_module(sd, nb, s[:, perm], z[:, perm][:, :, perm], m[:, perm], pm[:, perm][:, :, perm], dev, "bf16")
    keep = pm[0].bool()
    assert rel_l2(zp[0][keep[perm][:, perm]], za[0][perm][:, perm][keep[perm][:, perm]]) < 5e-3
    assert rel_l2(sp[0][m[0, perm].bool()], sa[0][perm][m[0, perm].bool()]) < 5e-3


def test_fully_masked_line_matches_reference(dev):
    """A line whose keys are all masked attends uniformly (finite), as the reference does."""
    n = 40
    sd = synthetic.make_weights(1, seed=3, std=0.05, with_s=False)
    _, z = synthetic.make_inputs(n, seed=2, with_s=False)
    pm = torch.ones(1, n, n)
    pm[0, 5, :] = 0
    pm[0, :, 7] = 0
    for precision, tol in (("fp32", 1e-4), ("bf16", 2e-2)):
        _, zo = run_module(sd, 1, None, z, None, pm, dev, precision, with_s=False)
        zr = orc.pairformer_stack(None, z[0], None, pm[0], sd, 1)[1]
        assert rel_l2(zo[0], zr) < tol, precision


# ---------------------------------------------------------------------------------------------
# benchmark configurations 2 and 3 at full size (bf16 tier)
# ---------------------------------------------------------------------------------------------
def test_cfg2_trimul_out_in_n512(dev):
    from tt_boltz_b200 import ops, weights
    n = 512
    sd = strip(synthetic.make_weights(1, seed=1, bf16_round=True, with_s=False))
    _, z = synthetic.make_inputs(n, seed=0, with_s=False, bf16_round=True)
    m, pm = synthetic.tail_padding_mask(n, 51)
    pm_u8 = (pm[0] != 0).to(torch.uint8).to(dev)
    ws = ops.Workspace(n, dev)
    zd = z[0].to(dev).clone()
    ops.tri_mul_bf16(zd, pm_u8, weights.pack_trimul(sd, "tri_mul_out.", dev), ws, False)
    ops.tri_mul_bf16(zd, pm_u8, weights.pack_trimul(sd, "tri_mul_in.", dev), ws, True)
    z1 = z[0] + orc.tri_mul(z[0], sd, "tri_mul_out", pm[0], False)
    z2 = z1 + orc.tri_mul(z1, sd, "tri_mul_in", pm[0], True)
    v = n - 51
    got = zd.cpu()
    assert rel_l2(got[:v, :v], z2[:v, :v]) < 2e-2
    assert rel_l2((got - z[0])[:v, :v], (z2 - z[0])[:v, :v]) < 2e-2      # the update itself
    # masked operands contribute exactly zero: re-run with garbage in the padded tokens
    z_g = z[0].clone()
    z_g[v:] = 100.0
    z_g[:, v:] = -100.0
    zd2 = z_g.to(dev).clone()
    ops.tri_mul_bf16(zd2, pm_u8, weights.pack_trimul(sd, "tri_mul_out.", dev), ws, False)
    ops.tri_mul_bf16(zd2, pm_u8, weights.pack_trimul(sd, "tri_mul_in.", dev), ws, True)
    assert torch.equal(zd2.cpu()[:v, :v], got[:v, :v])


def test_cfg3_triatt_start_end_n768(dev):
    from tt_boltz_b200 import ops, weights
    n = 768
    sd = strip(synthetic.make_weights(1, seed=1, bf16_round=True, with_s=False))
    _, z = synthetic.make_inputs(n, seed=0, with_s=False, bf16_round=True)
    for keep in (True, False):
        m, pm, _ = synthetic.chain_block_mask(n, 3, n_pad=32, seed=2, keep_inter_chain=keep)
        pm_u8 = (pm[0] != 0).to(torch.uint8).to(dev)
        ws = ops.Workspace(n, dev)
        zd = z[0].to(dev).clone()
        masks = ops.PairMasks(pm_u8)
        ops.tri_att_bf16(zd, masks, weights.pack_triatt(sd, "tri_att_start.", dev), ws, False)
        ops.tri_att_bf16(zd, masks, weights.pack_triatt(sd, "tri_att_end.", dev), ws, True)
        z1 = z[0] + orc.tri_att(z[0], sd, "tri_att_start", pm[0], False)
        z2 = z1 + orc.tri_att(z1, sd, "tri_att_end", pm[0], True)
        v = n - 32
        got = zd.cpu()
        assert torch.isfinite(got).all()
        assert rel_l2(got[:v, :v], z2[:v, :v]) < 2e-2
        assert rel_l2((got - z[0])[:v, :v], (z2 - z[0])[:v, :v]) < 2e-2


# ---------------------------------------------------------------------------------------------
# depth: error growth over a stack stays inside the bf16 tier
# ---------------------------------------------------------------------------------------------
def test_stack_depth_bf16(dev):
    n, nb = 64, 16
    sd = synthetic.make_weights(nb, seed=1)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 0)
    so, zo = run_module(sd, nb, s, z, m, pm, dev, "bf16")
    sr, zr = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, nb)
    assert rel_l2(zo[0], zr) < 2e-2
    assert rel_l2(so[0], sr) < 2e-2


def test_stack_64_blocks_bf16(dev):
    """The full trunk depth (64 blocks, independent N(0, 0.02) weights) stays inside the bf16 tier."""
    n, nb = 48, 64
    sd = synthetic.make_weights(nb, seed=1)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 5)
    so, zo = run_module(sd, nb, s, z, m, pm, dev, "bf16")
    sr, zr = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, nb)
    v = n - 5
    assert rel_l2(zo[0][:v, :v], zr[:v, :v]) < 2e-2
    assert rel_l2(so[0][:v], sr[:v]) < 2e-2


@pytest.mark.parametrize("precision,tol", [("fp32", 1e-4), ("bf16", 2e-2), ("mxfp8", 5e-2)])
@pytest.mark.parametrize("n", [1, 2, 3, 7, 33, 129])
def test_tiny_and_ragged_token_counts(dev, n, precision, tol):
    """Sizes below one tile, one past a tile boundary, and a single token, in every tier."""
    sd = synthetic.make_weights(1, seed=1, std=0.05, affine_jitter=0.3)
    s, z = synthetic.make_inputs(n, seed=n)
    npad = 1 if n > 2 else 0
    m, pm = synthetic.tail_padding_mask(n, npad)
    so, zo = run_module(sd, 1, s, z, m, pm, dev, precision)
    sr, zr = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, 1)
    v = n - npad
    assert rel_l2(zo[0][:v, :v], zr[:v, :v]) < tol
    assert rel_l2(so[0][:v], sr[:v]) < tol


def test_layer_forward_signature(dev):
    """PairformerLayer.forward(s, z, mask, pair_mask, chunk_size_tri_attn, use_kernels) returns new tensors."""
    n = 32
    sd = strip(synthetic.make_weights(1, seed=1))
    layer = B200PairformerLayer(384, 128, v2=True, precision="bf16")
    layer.load_state_dict(sd, strict=True)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.tail_padding_mask(n, 2)
    zd = z.to(dev)
    so, zo = layer(s.to(dev), zd, m.to(dev), pm.to(dev), 128, False)
    assert zo.shape == z.shape and so.shape == s.shape and zo.data_ptr() != zd.data_ptr()
    assert torch.equal(zd.cpu(), z)            # the caller's tensor is untouched


@pytest.mark.parametrize("nq,nk", [(1024, 1024), (128, 1024), (37, 300), (5, 132)])
def test_tensor_core_single_track_attention_agrees_with_direct_kernel(dev, nq, nk):
    """b200pf_f32_sattention picks the tensor-core kernel (3xTF32 products, one-pass softmax over staged key tiles)
    when its operands are 16-byte aligned and the direct-load SIMT kernel (two passes, fp32 FMAs) otherwise; both
    compute the same fp32 attention, so they agree to fp32 rounding: 2e-5 absolute on outputs of order 1."""
    import math
    from tt_boltz_b200._lib import call, ptr, stream
    heads, hd = 16, 24
    cs = heads * hd
    g = torch.Generator().manual_seed(nq * 7 + nk)
    pitch = (nk + 3) // 4 * 4
    qg = torch.randn(nq, 2 * cs, generator=g).to(dev)
    kvt = torch.randn(2 * cs, pitch, generator=g).to(dev)
    mask = (torch.rand(nk, generator=g) > 0.1).to(torch.uint8).to(dev)
    bias_qs = pitch                                            # padded rows keep the aligned path eligible for ragged nk
    bias_al = torch.randn(heads * nq * bias_qs + 4, generator=g).to(dev)
    bias_un = torch.empty_like(bias_al)
    bias_un[1:].copy_(bias_al[:-1])                            # same values, 4 bytes off alignment: forces the direct kernel
    outs = []
    for b in (bias_al, bias_un[1:]):
        o = torch.zeros(nq, cs, device=dev)
        call("b200pf_f32_sattention", ptr(qg), 2 * cs, qg.data_ptr() + 4 * cs, 2 * cs, ptr(kvt), kvt.data_ptr() + 4 * cs * pitch, pitch,
             ptr(o), cs, b.data_ptr(), nq * bias_qs, bias_qs, ptr(mask), nq, nk, heads, hd, 1.0 / math.sqrt(hd), 1e6, stream())
        outs.append(o)
    torch.cuda.synchronize()
    assert bias_al.data_ptr() % 16 == 0 and bias_un[1:].data_ptr() % 16 == 4
    assert torch.isfinite(outs[0]).all()
    assert (outs[0] - outs[1]).abs().max().item() < 2e-5


@pytest.mark.parametrize("n, amp", [(200, 40.0), (320, 30.0)])
def test_attention_core_with_scores_that_jump_far_above_the_running_reference(dev, n, amp):
    """The core alone, on synthetic q / k / v / bias whose scores (log2 domain) span hundreds of units, so that within a
    line a later key tile lies far more than 2^64 above everything seen before: the one-pass softmax has to notice
    before it releases the scores and redo such a tile with a fresh reference.  Against a float64 softmax of the same
    bf16 inputs; tolerance = the rounding of p to bf16 (2^-9 relative per term)."""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import call, ptr, stream
    g = torch.Generator().manual_seed(21)
    heads, hd, lines = 4, 32, 9
    pitch = (n + 7) // 8 * 8
    mpitch = (n + 63) // 64 * 64
    q = torch.randn(lines, n, heads, hd, generator=g).bfloat16()
    k = (torch.randn(lines, n, heads, hd, generator=g) * amp / (hd ** 0.5)).bfloat16()
    # keys later in the line are systematically larger: the running maximum keeps growing in big steps
    k = (k.float() * torch.linspace(0.05, 1.0, n)[None, :, None, None] ** 2).bfloat16()
    v = torch.randn(lines, n, heads, hd, generator=g).bfloat16()
    bias = (torch.randn(n, heads, n, generator=g) * 3).bfloat16()           # [query][head][key]
    mask = (torch.rand(lines, n, generator=g) > 0.1)
    mask[:, 0] = True
    vt = torch.zeros(lines, heads, hd, pitch, dtype=torch.bfloat16)
    vt[..., :n] = v.permute(0, 2, 3, 1)
    bias_p = torch.zeros(n, heads, pitch, dtype=torch.bfloat16)
    bias_p[..., :n] = bias
    mask_p = torch.zeros(lines, mpitch, dtype=torch.uint8)
    mask_p[:, :n] = mask.to(torch.uint8)
    o = torch.zeros(lines, n, heads * hd, dtype=torch.bfloat16, device=dev)
    qd, kd, vtd, bd, md = q.to(dev).contiguous(), k.to(dev).contiguous(), vt.to(dev), bias_p.to(dev), mask_p.to(dev)
    call("b200pf_triatt_core_tc4", ptr(qd), ptr(kd), ptr(vtd), pitch, ptr(bd), pitch, heads * pitch, ptr(md), mpitch,
         ptr(o), n * heads * hd, heads * hd, lines, n, stream())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    s = torch.einsum("lqhd,lkhd->lhqk", q.double(), k.double()) + bias.double().permute(1, 0, 2)[None]
    s = s + torch.where(mask, 0.0, -1.0e9 * 1.4426950408889634)[:, None, None, :].double()
    span = float((s.amax(-1) - s[..., : 64].amax(-1)).max())
    assert span > 100, span                                                  # the premise: far beyond the 2^64 headroom
    p = torch.exp2(s - s.amax(-1, keepdim=True))
    want = torch.einsum("lhqk,lkhd->lqhd", p / p.sum(-1, keepdim=True), v.double()).reshape(lines, n, heads * hd)
    got = o.cpu().double()
    assert torch.isfinite(got).all()
    assert rel_l2(got, want) < 6e-3
