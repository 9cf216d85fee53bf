"""CPU (fp32, gloo) restatement of the row-sharded block: the same exchanges as
tt_boltz_b200/sharded.py, with the oracle's formulas on the local pieces.  Test infrastructure."""
import math

import torch

from oracle import pairformer_oracle as orc
from tt_boltz_b200.sharded import all_gather_cat, all_to_all_blocks, cols_to_rows, rows_to_cols


def _gated(z, w, pre, mask):
    x = orc._ln(z, w, pre + ".norm_in")
    u = orc._lin(x, w, pre + ".p_in") * torch.sigmoid(orc._lin(x, w, pre + ".g_in")) * mask[..., None]
    return x, u


def _channel_parallel_contract(a_pl, b_pl, world, contract_rows):
    """a_pl, b_pl: channel-major planes [D][plane rows][plane cols] of this rank's shard.  All-to-all to channel
    shards, contract D/P channels for every row, all-to-all the result back to row shards: [D][nr][N]."""
    d = a_pl.shape[0]
    cl = d // world
    a_ch = all_to_all_blocks(a_pl.reshape(world, -1)).view(world, cl, a_pl.shape[1], a_pl.shape[2])   # [src][cl][rows][cols]
    b_ch = all_to_all_blocks(b_pl.reshape(world, -1)).view(world, cl, b_pl.shape[1], b_pl.shape[2])
    if contract_rows:      # incoming: the source rank owns a block of the contraction index (plane columns)
        a_f = a_ch.permute(1, 2, 0, 3).reshape(cl, a_pl.shape[1], -1)       # [cl][i][k]
        b_f = b_ch.permute(1, 2, 0, 3).reshape(cl, b_pl.shape[1], -1)
    else:                  # outgoing: the source rank owns a block of the operand's rows
        a_f = a_ch.permute(1, 0, 2, 3).reshape(cl, -1, a_pl.shape[2])       # [cl][i][k]
        b_f = b_ch.permute(1, 0, 2, 3).reshape(cl, -1, b_pl.shape[2])
    x = torch.einsum("cik,cjk->cij", a_f, b_f)                               # [cl][N][N]
    n = x.shape[1]
    nr = n // world
    send = x.view(cl, world, nr, n).permute(1, 0, 2, 3).contiguous()         # [dest][cl][nr][N]
    return all_to_all_blocks(send.view(world, -1)).view(d, nr, n)            # [src * cl + c][nr][N]


def _tri_mul_out(z_loc, w, pre, mask_loc, world):
    nr, n, _ = z_loc.shape
    x, u = _gated(z_loc, w, pre, mask_loc)
    d = u.shape[-1] // 2
    a_pl = u[..., :d].permute(2, 0, 1).contiguous()                           # [D][i local][k]
    b_pl = u[..., d:].permute(2, 0, 1).contiguous()                           # [D][j local][k]
    t = _channel_parallel_contract(a_pl, b_pl, world, False).permute(1, 2, 0)
    return z_loc + orc._lin(orc._ln(t, w, pre + ".norm_out"), w, pre + ".p_out") * torch.sigmoid(orc._lin(x, w, pre + ".g_out"))


def _tri_mul_in(z_loc, w, pre, mask_loc, world):
    nr, n, _ = z_loc.shape
    x, u = _gated(z_loc, w, pre, mask_loc)
    d = u.shape[-1] // 2
    a_pl = u[..., :d].permute(2, 1, 0).contiguous()                           # [D][i][k local]
    b_pl = u[..., d:].permute(2, 1, 0).contiguous()                           # [D][j][k local]
    t = _channel_parallel_contract(a_pl, b_pl, world, True).permute(1, 2, 0)
    return z_loc + orc._lin(orc._ln(t, w, pre + ".norm_out"), w, pre + ".p_out") * torch.sigmoid(orc._lin(x, w, pre + ".g_out"))


def _attend(x, beta_all, mask_lines, w, pre):
    """x [lines][pos][C] normalised input; beta_all [q][k][H]; mask_lines [lines][pos]."""
    lines, n, _ = x.shape
    heads = beta_all.shape[-1]
    q = orc._lin(x, w, pre + ".mha.linear_q")
    hd = q.shape[-1] // heads
    q = q.view(lines, n, heads, hd) / math.sqrt(hd)
    k = orc._lin(x, w, pre + ".mha.linear_k").view(lines, n, heads, hd)
    v = orc._lin(x, w, pre + ".mha.linear_v").view(lines, n, heads, hd)
    g = orc._lin(x, w, pre + ".mha.linear_g")
    a = torch.einsum("iqhd,ikhd->ihqk", q, k)
    a = a + (orc.TRI_ATT_INF * (mask_lines - 1))[:, None, None, :]
    a = a + beta_all.permute(2, 0, 1)[None]
    a = torch.softmax(a, -1)
    o = torch.einsum("ihqk,ikhd->iqhd", a, v).reshape(lines, n, heads * hd) * torch.sigmoid(g)
    return orc._lin(o, w, pre + ".mha.linear_o")


def _tri_att_start(z_loc, w, pre, mask_loc):
    nr, n, _ = z_loc.shape
    x = orc._ln(z_loc, w, pre + ".layer_norm")
    beta_all = all_gather_cat(orc._lin(x, w, pre + ".linear")).view(n, n, -1)            # [q][k][H]
    return z_loc + _attend(x, beta_all, mask_loc, w, pre)


def _tri_att_end(z_loc, w, pre, pm, r0):
    nr, n, _ = z_loc.shape
    zc = rows_to_cols(z_loc)                                                             # [i][j local][C]
    xc = orc._ln(zc, w, pre + ".layer_norm")
    beta_loc = orc._lin(xc, w, pre + ".linear").permute(1, 0, 2).contiguous()            # [q = col local][k = row][H]
    beta_all = all_gather_cat(beta_loc).view(n, n, -1)
    mask_lines = pm[:, r0:r0 + nr].transpose(0, 1)                                        # [line j][key i']
    upd = _attend(xc.transpose(0, 1).contiguous(), beta_all, mask_lines, w, pre)          # [line j][pos i][C]
    return cols_to_rows((zc + upd.transpose(0, 1)).contiguous())


def sharded_block_cpu(w, pre, s, z_loc, mask, pm, rank, world, num_heads=16):
    nr, n, _ = z_loc.shape
    r0 = rank * nr
    mask_loc = pm[r0:r0 + nr]
    z_loc = _tri_mul_out(z_loc, w, pre + "tri_mul_out", mask_loc, world)
    z_loc = _tri_mul_in(z_loc, w, pre + "tri_mul_in", mask_loc, world)
    z_loc = _tri_att_start(z_loc, w, pre + "tri_att_start", mask_loc)
    z_loc = _tri_att_end(z_loc, w, pre + "tri_att_end", pm, r0)
    z_loc = z_loc + orc.transition(z_loc, w, pre + "transition_z")
    # single track: attention for local query rows only, then gather the gated outputs
    cs = s.shape[1]
    hd = cs // num_heads
    ap = pre + "attention"
    sn = orc._ln(s, w, pre + "pre_norm_s")
    q = orc._lin(sn[r0:r0 + nr], w, ap + ".proj_q").view(nr, num_heads, hd)
    g = torch.sigmoid(orc._lin(sn[r0:r0 + nr], w, ap + ".proj_g"))
    k = orc._lin(sn, w, ap + ".proj_k").view(n, num_heads, hd)
    v = orc._lin(sn, w, ap + ".proj_v").view(n, num_heads, hd)
    bias = orc._lin(orc._ln(z_loc, w, ap + ".proj_z.0"), w, ap + ".proj_z.1").permute(2, 0, 1)
    att = torch.einsum("ihd,jhd->hij", q, k) / (hd ** 0.5) + bias + ((1 - mask) * -orc.S_ATT_INF)[None, None, :]
    o = torch.einsum("hij,jhd->ihd", att.softmax(-1), v).reshape(nr, cs)
    s_loc = s[r0:r0 + nr] + orc._lin((g * o).contiguous(), w, ap + ".proj_o")
    s_loc = s_loc + orc.transition(s_loc, w, pre + "transition_s")
    s = all_gather_cat(s_loc.contiguous()).view(n, cs)
    return s, z_loc
