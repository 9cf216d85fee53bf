"""MXFP8 triangle multiplication (e4m3 values, e8m0 scale per 32 along the contraction index).

The reference's block-fp8 mode (tt_bio/tenstorrent.py:178-181) has no bit pattern to match - its
format is a different block float - so these tests pin (1) the format itself: scale rule, scale
layout and value bytes written by the producer, decoded here with torch; (2) the block-scaled
tensor-core contraction against an fp32 einsum over the decoded operands and against the bf16
contraction fed the (exactly) expanded operands; (3) the whole layer / stack against the fp32
oracle at the 5e-2 tier.
"""
import ctypes as C

import pytest
import torch

from oracle import pairformer_oracle as orc
from tests.conftest import rel_l2
from tt_boltz_b200 import B200PairformerModule, synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def decode_scales(scales: torch.Tensor, rows: int, cols: int, channels: int = 128) -> torch.Tensor:
    """[channels][rows][ceil(cols/32)] e8m0 bytes out of the 512-byte block layout of include/b200pf.h."""
    kgroups, row_blocks = (cols + 127) // 128, 2 * ((rows + 255) // 256)
    nkb = (cols + 31) // 32
    d = torch.arange(channels).view(-1, 1, 1)
    r = torch.arange(rows).view(1, -1, 1)
    kb = torch.arange(nkb).view(1, 1, -1)
    off = ((d * kgroups + kb // 4) * row_blocks + r // 128) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    return scales.cpu()[off.reshape(-1)].view(channels, rows, nkb)


def decode_planes(vals: torch.Tensor, scales: torch.Tensor, rows: int, cols: int, pitch: int):
    """fp32 [128][rows][cols] operand, raw e4m3 magnitudes and scale bytes."""
    q = vals.cpu()[: 128 * rows * pitch].view(128, rows, pitch)[:, :, :cols].contiguous().view(torch.float8_e4m3fn).float()
    e = decode_scales(scales, rows, cols).to(torch.int32)
    sc = torch.pow(2.0, (e.clamp(min=1) - 127).float()).repeat_interleave(32, dim=2)[:, :, :cols]
    return q * sc, q, e


def run_producer(dev, n, incoming, seed=0):
    from tt_boltz_b200 import ops, weights
    from tt_boltz_b200._lib import call, ptr, stream
    sd = synthetic.make_weights(1, seed=seed + 1, std=0.05, affine_jitter=0.3)
    sd = {k[len("layers.0."):]: v for k, v in sd.items() if k.startswith("layers.0.")}
    _, z = synthetic.make_inputs(n, seed=seed, with_s=False)
    _, pm = synthetic.tail_padding_mask(n, 5)
    name = "tri_mul_in." if incoming else "tri_mul_out."
    w = weights.pack_trimul(sd, name, dev)
    ws = ops.Workspace(n, dev)
    zd = z[0].to(dev).contiguous()
    pmd = pm[0].to(torch.uint8).to(dev).contiguous()
    return sd, z, pm, w, ws, zd, pmd


@pytest.mark.parametrize("n,incoming", [(40, False), (128, True), (200, False), (300, True)])
def test_producer_writes_the_documented_format(dev, n, incoming):
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import PlaneOut, call, ptr, stream
    sd, z, pm, w, ws, zd, pmd = run_producer(dev, n, incoming)
    pitch8 = (n + 15) // 16 * 16
    a8, b8 = ws.buf[3].view(torch.uint8), ws.buf[4].view(torch.uint8)
    a8.fill_(0x7F)          # NaN pattern: anything left unwritten inside the valid region shows up
    b8.fill_(0x7F)
    sa, sb = ws.mx_scales()
    call("b200pf_trimul_producer_mx", ptr(zd), ptr(pmd), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]),
         ptr(a8), ptr(b8), ptr(sa), ptr(sb), n * pitch8, pitch8, n, n, int(incoming), stream())
    # the same operands from the bf16 producer
    a16, b16 = ws.buf[0], ws.buf[1]
    oa, ob = PlaneOut(ptr(a16), ws.plane_stride, 0, 0), PlaneOut(ptr(b16), ws.plane_stride, 0, 0)
    call("b200pf_trimul_producer", ptr(zd), ptr(pmd), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]),
         C.byref(oa), C.byref(ob), ws.pitch, n, n, int(incoming), stream())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for v8, sc, v16 in ((a8, sa, a16), (b8, sb, b16)):
        deq, q, e = decode_planes(v8, sc, n, n, pitch8)
        ref = v16.cpu()[: 128 * n * ws.pitch].view(128, n, ws.pitch)[:, :, :n].float()
        assert torch.isfinite(deq).all()
        err = rel_l2(deq, ref)
        assert 1e-3 < err < 5e-2, err                      # quantised, and no worse than e4m3 allows
        # scale rule: the largest magnitude of every non-zero block lies in [224, 448] (224 < amax/scale <= 448, rounded)
        pad = (-n) % 32
        qa = torch.nn.functional.pad(q.abs(), (0, pad)).view(128, n, -1, 32).amax(dim=3)
        nz = qa > 0
        assert (qa[nz] <= 448).all() and (qa[nz] >= 224).all()
        assert (e[~nz] == 0).all()                         # blocks of zeros (masked positions) carry scale byte 0
        # masked positions are exactly zero
        keep = pm[0].bool()
        keep = keep.t() if incoming else keep
        assert (deq[:, ~keep] == 0).all()


@pytest.mark.parametrize("n", [24, 100, 128, 264, 512])
def test_block_scaled_contraction(dev, n):
    """variant 2 against an fp32 einsum of the decoded operands and against expand -> bf16 contraction."""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import Planes, call, ptr, stream
    lib = _lib.load()
    pitch8, pitch = (n + 15) // 16 * 16, (n + 7) // 8 * 8
    g = torch.Generator().manual_seed(n)
    nkb = (n + 31) // 32
    ops_dev, ops_f32, scales_dev = [], [], []
    for _ in range(2):
        q = (torch.randn(128, n, pitch8, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
        q.view(torch.uint8)[:, :, n:] = 0
        e = torch.randint(110, 135, (128, n, nkb), generator=g, dtype=torch.int32)
        e[:, ::7, :] = 127
        nbytes = lib.b200pf_mx_scale_bytes(n, n, 128)
        flat = torch.zeros(nbytes, dtype=torch.uint8)
        kgroups, row_blocks = (n + 127) // 128, 2 * ((n + 255) // 256)
        d = torch.arange(128).view(-1, 1, 1)
        r = torch.arange(n).view(1, -1, 1)
        kb = torch.arange(nkb).view(1, 1, -1)
        off = ((d * kgroups + kb // 4) * row_blocks + r // 128) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
        flat[off.reshape(-1)] = e.to(torch.uint8).reshape(-1)
        ops_dev.append(q.view(torch.uint8).to(dev))
        scales_dev.append(flat.to(dev))
        sc = torch.pow(2.0, (e - 127).float()).repeat_interleave(32, dim=2)[:, :, :n]
        ops_f32.append(q[:, :, :n].float() * sc)
    ref = torch.einsum("dik,djk->dij", ops_f32[0].to(dev), ops_f32[1].to(dev)).cpu()
    x2 = torch.zeros(128, n, pitch, dtype=torch.bfloat16, device=dev)
    pa = Planes(ptr(ops_dev[0]), n * pitch8, 0, pitch8, n, n, 1, 0)
    pb = Planes(ptr(ops_dev[1]), n * pitch8, 0, pitch8, n, n, 1, 0)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), ptr(scales_dev[0]), ptr(scales_dev[1]), ptr(x2), n * pitch, pitch,
         0, 0, 128, 2, stream())
    # expand to bf16 (exact) and contract with the bf16 kernel
    exp = [torch.zeros(128, n, pitch, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    for i in range(2):
        call("b200pf_mx_dequant", ptr(ops_dev[i]), ptr(scales_dev[i]), ptr(exp[i]), n * pitch8, pitch8, n * pitch, pitch, n, n, 128,
             stream())
    x0 = torch.zeros(128, n, pitch, dtype=torch.bfloat16, device=dev)
    pa0 = Planes(ptr(exp[0]), n * pitch, 0, pitch, n, n, 1, 0)
    pb0 = Planes(ptr(exp[1]), n * pitch, 0, pitch, n, n, 1, 0)
    call("b200pf_trimul_contract", C.byref(pa0), C.byref(pb0), None, None, ptr(x0), n * pitch, pitch, 0, 0, 128, 0, stream())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for i in range(2):
        assert torch.equal(exp[i][:, :, :n].float().cpu(), ops_f32[i]), "expansion to bf16 must be exact"
    assert rel_l2(x0[:, :, :n].float().cpu(), ref) < 4e-3
    assert rel_l2(x2[:, :, :n].float().cpu(), ref) < 4e-3
    assert rel_l2(x2[:, :, :n].float().cpu(), x0[:, :, :n].float().cpu()) < 1e-3


def _encode_scales(e: torch.Tensor, rows: int, cols: int, channels: int, nbytes: int) -> torch.Tensor:
    """e [channels][rows][ceil(cols/32)] scale bytes -> the 512-byte block layout."""
    nkb = (cols + 31) // 32
    kgroups, row_blocks = (cols + 127) // 128, 2 * ((rows + 255) // 256)
    d = torch.arange(channels).view(-1, 1, 1)
    r = torch.arange(rows).view(1, -1, 1)
    kb = torch.arange(nkb).view(1, 1, -1)
    off = ((d * kgroups + kb // 4) * row_blocks + r // 128) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    flat = torch.zeros(nbytes, dtype=torch.uint8)
    flat[off.reshape(-1)] = e.to(torch.uint8).reshape(-1)
    return flat


@pytest.mark.parametrize("seg_is_k", [0, 1])
@pytest.mark.parametrize("world,nr", [(2, 128), (3, 128), (2, 256)])
def test_block_scaled_contraction_segmented_operands_and_grouped_output(dev, seg_is_k, world, nr):
    """The layouts of the sharded MXFP8 triangle multiplication: operands in `world` segments (blocks of rows or of
    the contraction index), each with its own scale buffer packed behind the previous one, the result written in
    groups of nr output rows.  Against an fp32 einsum of the decoded operands.  (world 3 x 128 rows: an odd number
    of 128-row blocks, so the last 256-row B tile has no upper half.)"""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import Planes, call, ptr, stream
    lib = _lib.load()
    cl, n = 8, world * nr
    g = torch.Generator().manual_seed(5 * world + seg_is_k)
    rows, cols = (n, nr) if seg_is_k else (nr, n)
    sf_seg = lib.b200pf_mx_scale_bytes(rows, cols, cl)
    full, vals, scales = [], [], []
    for _ in range(2):
        q = (torch.randn(cl, n, n, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
        e = torch.randint(118, 132, (cl, n, n // 32), generator=g, dtype=torch.int32)
        full.append(q.float() * torch.pow(2.0, (e - 127).float()).repeat_interleave(32, dim=2))
        qb = q.view(torch.uint8)
        if seg_is_k:     # segment s: k in [s*nr, (s+1)*nr), all rows
            v = qb.view(cl, n, world, nr).permute(2, 0, 1, 3).contiguous()
            sc = torch.cat([_encode_scales(e[:, :, s * (nr // 32):(s + 1) * (nr // 32)], n, nr, cl, sf_seg) for s in range(world)])
        else:            # segment s: rows [s*nr, (s+1)*nr), all k
            v = qb.view(cl, world, nr, n).permute(1, 0, 2, 3).contiguous()
            sc = torch.cat([_encode_scales(e[:, s * nr:(s + 1) * nr], nr, n, cl, sf_seg) for s in range(world)])
        vals.append(v.to(dev))
        scales.append(sc.to(dev))
    ref = torch.einsum("cik,cjk->cij", full[0].to(dev), full[1].to(dev)).cpu()
    x = torch.zeros(world, cl, nr, n, dtype=torch.bfloat16, device=dev)            # [group = i / nr][c][i local][j]
    pa = Planes(ptr(vals[0]), rows * cols, cl * rows * cols, cols, rows, cols, world, seg_is_k)
    pb = Planes(ptr(vals[1]), rows * cols, cl * rows * cols, cols, rows, cols, world, seg_is_k)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), ptr(scales[0]), ptr(scales[1]), ptr(x), nr * n, n, nr, cl * nr * n, cl, 2, stream())
    assert _lib.device_status() == 0
    got = x.permute(1, 0, 2, 3).reshape(cl, n, n).float().cpu()
    assert rel_l2(got, ref) < 4e-3


def _run(sd, blocks, s, z, m, pm, dev, precision, **attrs):
    mod = B200PairformerModule(384, 128, blocks, v2=True, precision=precision)
    mod.load_state_dict(sd, strict=True)
    for layer in mod.layers:
        for k, v in attrs.items():
            setattr(layer, k, v)
    s2, z2 = mod(s.to(dev), z.to(dev), m.to(dev), pm.to(dev))
    return s2.float().cpu(), z2.float().cpu()


def test_layer_mxfp8_against_oracle_and_cross_check(dev):
    n = 136
    sd = synthetic.make_weights(1, seed=1, std=0.05, affine_jitter=0.3)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = synthetic.random_padding_mask(n, 0.05, seed=3)
    s_mx, z_mx = _run(sd, 1, s, z, m, pm, dev, "mxfp8")
    s_x, z_x = _run(sd, 1, s, z, m, pm, dev, "mxfp8", mx_contract_variant=0)
    s_ref, z_ref = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, 1)
    keep = pm[0].bool()
    assert rel_l2((z_mx - z)[0][keep], (z_x - z)[0][keep]) < 5e-3          # the two contractions agree
    assert rel_l2(z_mx[0][keep], z_ref[keep]) < 5e-2
    assert rel_l2((z_mx - z)[0][keep], (z_ref - z[0])[keep]) < 5e-2         # also on the update alone
    assert rel_l2(s_mx[0][m[0].bool()], s_ref[m[0].bool()]) < 5e-2


def test_stack_mxfp8_tier(dev):
    """16 blocks at N = 96 with 5 % random padding: inside the 5e-2 tier, and really quantised."""
    n, blocks = 96, 16
    sd = synthetic.make_weights(blocks, seed=7)
    s, z = synthetic.make_inputs(n, seed=8)
    m, pm = synthetic.random_padding_mask(n, 0.05, seed=3)
    s_mx, z_mx = _run(sd, blocks, s, z, m, pm, dev, "mxfp8")
    s_bf, z_bf = _run(sd, blocks, s, z, m, pm, dev, "bf16")
    s_ref, z_ref = orc.pairformer_stack(s[0], z[0], m[0], pm[0], sd, blocks)
    keep = pm[0].bool()
    e_mx, e_bf = rel_l2(z_mx[0][keep], z_ref[keep]), rel_l2(z_bf[0][keep], z_ref[keep])
    assert e_mx < 5e-2, e_mx
    assert e_mx > e_bf
    assert rel_l2(s_mx[0][m[0].bool()], s_ref[m[0].bool()]) < 5e-2
