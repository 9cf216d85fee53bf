"""Row-sampled CPU timing of one Pairformer block with the oracle's formulas (TEST / BENCH
INFRASTRUCTURE, not product code).

A full fp32 block at N = 1024 costs tens of seconds on a host CPU.  Every sub-operation of the
block is a sum of equal-cost pieces over the rows i of its output, so timing the pieces for R
sampled rows and scaling by N / R estimates the whole block.  What a sampled row needs from
*other* rows (the k-side operand b of the triangle multiplication, the triangle bias of all
pairs) is computed outside the timed region: in a full run that work is attributed to the rows
that own it, so each row's share is counted exactly once.

``block_rows`` returns the updated rows so that tests can check them against the full oracle.
"""
from __future__ import annotations

import math
import time
from typing import Dict, Tuple

import torch

from . import pairformer_oracle as orc

Tensor = torch.Tensor


def _gated_in(z_rows: Tensor, w, pre: str, mask_rows: Tensor) -> Tuple[Tensor, Tensor]:
    x = orc._ln(z_rows, w, pre + ".norm_in")
    u = orc._lin(x, w, pre + ".p_in") * torch.sigmoid(orc._lin(x, w, pre + ".g_in"))
    return x, u * mask_rows[..., None]


def tri_mul_rows(z: Tensor, w, pre: str, pm: Tensor, incoming: bool, rows: Tensor) -> Tuple[Tensor, float]:
    d = w[pre + ".p_out.weight"].shape[1]
    others = torch.ones(z.shape[0], dtype=torch.bool)
    others[rows] = False
    _, u_other = _gated_in(z[others], w, pre, pm[others])              # untimed: owned by other rows
    t0 = time.perf_counter()
    x_r, u_r = _gated_in(z[rows], w, pre, pm[rows])
    u_all = torch.empty(z.shape[0], z.shape[1], 2 * d)
    u_all[rows] = u_r
    u_all[others] = u_other
    a, b = u_all[..., :d], u_all[..., d:]
    if incoming:
        t = torch.einsum("kic,kjc->ijc", a[:, rows], b)
    else:
        t = torch.einsum("ikc,jkc->ijc", a[rows], b)
    upd = orc._lin(orc._ln(t, w, pre + ".norm_out"), w, pre + ".p_out") * torch.sigmoid(orc._lin(x_r, w, pre + ".g_out"))
    out = z[rows] + upd
    return out, time.perf_counter() - t0


def tri_att_rows(z: Tensor, w, pre: str, pm: Tensor, ending: bool, rows: Tensor) -> Tuple[Tensor, float]:
    """Rows of the starting-node update, or columns (returned as rows of z transposed) of the ending one."""
    n = z.shape[0]
    zt, pmt = (z.transpose(0, 1), pm.transpose(0, 1)) if ending else (z, pm)
    others = torch.ones(n, dtype=torch.bool)
    others[rows] = False
    beta_other = orc._lin(orc._ln(zt[others], w, pre + ".layer_norm"), w, pre + ".linear")   # untimed
    t0 = time.perf_counter()
    zr = zt[rows].contiguous()                                       # includes the transposition copy
    x = orc._ln(zr, w, pre + ".layer_norm")
    beta = torch.empty(n, n, beta_other.shape[-1])
    beta[rows] = orc._lin(x, w, pre + ".linear")
    beta[others] = beta_other
    heads = beta.shape[-1]
    q = orc._lin(x, w, pre + ".mha.linear_q")
    hd = q.shape[-1] // heads
    r = len(rows)
    q = q.view(r, n, heads, hd) / math.sqrt(hd)
    k = orc._lin(x, w, pre + ".mha.linear_k").view(r, n, heads, hd)
    v = orc._lin(x, w, pre + ".mha.linear_v").view(r, n, heads, hd)
    g = orc._lin(x, w, pre + ".mha.linear_g")
    a = torch.einsum("iqhd,ikhd->ihqk", q, k)
    a = a + (orc.TRI_ATT_INF * (pmt[rows] - 1))[:, None, None, :]
    a = a + beta.permute(2, 0, 1)[None]
    a = torch.softmax(a, dim=-1)
    o = torch.einsum("ihqk,ikhd->iqhd", a, v).reshape(r, n, heads * hd) * torch.sigmoid(g)
    out = zr + orc._lin(o, w, pre + ".mha.linear_o")
    return out, time.perf_counter() - t0


def transition_rows(z: Tensor, w, pre: str, rows: Tensor) -> Tuple[Tensor, float]:
    t0 = time.perf_counter()
    zr = z[rows]
    out = zr + orc.transition(zr, w, pre)
    return out, time.perf_counter() - t0


def sampled_block_seconds(s: Tensor, z: Tensor, mask: Tensor, pm: Tensor, w: Dict[str, Tensor], pre: str,
                          n_rows: int, seed: int = 0, num_heads: int = 16) -> Dict[str, float]:
    """Estimated seconds of one full block from ``n_rows`` sampled rows (single track timed in full)."""
    n = z.shape[0]
    g = torch.Generator().manual_seed(seed)
    rows = torch.sort(torch.randperm(n, generator=g)[:n_rows]).values
    scale = n / float(n_rows)
    out: Dict[str, float] = {}
    with torch.no_grad():
        out["tri_mul_out"] = tri_mul_rows(z, w, pre + "tri_mul_out", pm, False, rows)[1] * scale
        out["tri_mul_in"] = tri_mul_rows(z, w, pre + "tri_mul_in", pm, True, rows)[1] * scale
        out["tri_att_start"] = tri_att_rows(z, w, pre + "tri_att_start", pm, False, rows)[1] * scale
        out["tri_att_end"] = tri_att_rows(z, w, pre + "tri_att_end", pm, True, rows)[1] * scale
        out["transition_z"] = transition_rows(z, w, pre + "transition_z", rows)[1] * scale
        t0 = time.perf_counter()
        s_n = orc._ln(s, w, pre + "pre_norm_s")
        s2 = s + orc.attention_pair_bias(s_n, z, mask, w, pre + "attention", num_heads)
        s2 = s2 + orc.transition(s2, w, pre + "transition_s")
        out["single_track"] = time.perf_counter() - t0
    out["total"] = sum(out.values())
    return out
