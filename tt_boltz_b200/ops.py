"""Host orchestration of the Pairformer sub-operations on one GPU.

Each function enqueues b200pf kernels (through the C ABI) on torch's current stream and updates
the fp32 residual tensor in place.  Tensors here are B = 1 folded away: z [N, N, 128] fp32,
s [N, 384] fp32, masks uint8.  Nothing in this file computes on the CPU or with torch math.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional

import torch

from . import _lib
from ._lib import PlaneOut, Planes, call, ptr, stream

C_Z = 128


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class PairMasks:
    """uint8 forms of the pair mask: [N][N] for the triangle multiplication, and one contiguous,
    64-padded row per attention line for the starting (rows) and ending (columns) node."""

    def __init__(self, pair_mask_u8: torch.Tensor) -> None:
        n = pair_mask_u8.shape[0]
        self.n = n
        self.pitch = _round_up(n, 64)
        self.pm = pair_mask_u8.contiguous()
        self.rows = torch.zeros(n, self.pitch, dtype=torch.uint8, device=pair_mask_u8.device)
        self.rows[:, :n] = self.pm
        self.cols = torch.zeros(n, self.pitch, dtype=torch.uint8, device=pair_mask_u8.device)
        self.cols[:, :n] = self.pm.t()


class Workspace:
    """bf16 scratch for one token count: five [N*pitch*128] buffers shared by the sub-operations
    (triangle multiplication uses three as a / b / x planes, triangle attention five as
    q / k / v / g / o), plus the triangle-bias tile source [4][N][pitch]."""

    def __init__(self, n: int, device) -> None:
        self.n = n
        self.pitch = _round_up(n, 8)
        self.plane_stride = n * self.pitch
        elems = C_Z * self.plane_stride
        self.buf = [torch.empty(elems, dtype=torch.bfloat16, device=device) for _ in range(5)]
        self.tri_bias = torch.empty(4 * n * self.pitch, dtype=torch.bfloat16, device=device)
        self._mx_scales = None

    def mx_scales(self):
        """Two zero-initialised e8m0 scale buffers (a and b operand) for the MXFP8 triangle multiplication."""
        if self._mx_scales is None:
            nbytes = _lib.load().b200pf_mx_scale_bytes(self.n, self.n, C_Z)
            self._mx_scales = [torch.zeros(nbytes, dtype=torch.uint8, device=self.buf[0].device) for _ in range(2)]
        return self._mx_scales


# ------------------------------------------------------------------------------------------------
# bf16 tier (fused kernels)
# ------------------------------------------------------------------------------------------------
def trimul_producer_weights(w: Dict[str, torch.Tensor]):
    """(ln_gamma, ln_beta, w_pg) pointers of the triangle-multiplication producer."""
    return ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"])


def triatt_producer_weights(w: Dict[str, torch.Tensor]):
    """(ln_gamma, ln_beta, w_bias_f32, w_qkgv) pointers of the triangle-attention producer."""
    return ptr(w["ln_gamma"]), ptr(w["ln_beta"]), ptr(w["w_bias_f32"]), ptr(w["w_qkgv_tc"])


def trimul_epilogue(z, x, plane_stride, pitch, w, rows, n) -> None:
    call("b200pf_trimul_epilogue_tc", ptr(z), ptr(x), plane_stride, pitch, ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]),
         ptr(w["w_pout_tc"]), ptr(w["w_gout_tc"]), ptr(w["wsum_tc"]), ptr(w["wb_tc"]), rows, n, stream())


def tri_mul_bf16(z: torch.Tensor, mask_u8: torch.Tensor, w: Dict[str, torch.Tensor], ws: Workspace,
                 incoming: bool, before_z_write=None) -> None:
    """``before_z_write`` is called (if given) right before the first kernel that writes z, the epilogue."""
    n = z.shape[0]
    a, b, x = ws.buf[0], ws.buf[1], ws.buf[2]
    st = stream()
    oa = PlaneOut(ptr(a), ws.plane_stride, 0, 0)
    ob = PlaneOut(ptr(b), ws.plane_stride, 0, 0)
    call("b200pf_trimul_producer", ptr(z), ptr(mask_u8), *trimul_producer_weights(w), C.byref(oa), C.byref(ob),
         ws.pitch, n, n, int(incoming), st)
    pa = Planes(ptr(a), ws.plane_stride, 0, ws.pitch, n, n, 1, 0)
    pb = Planes(ptr(b), ws.plane_stride, 0, ws.pitch, n, n, 1, 0)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), ws.plane_stride, ws.pitch,
         0, 0, C_Z, 0, st)
    if before_z_write is not None:
        before_z_write()
    trimul_epilogue(z, x, ws.plane_stride, ws.pitch, w, n, n)


def tri_mul_mxfp8(z: torch.Tensor, mask_u8: torch.Tensor, w: Dict[str, torch.Tensor], ws: Workspace,
                  incoming: bool, contract_variant: int = 2, before_z_write=None) -> None:
    """Triangle multiplication with MXFP8 operands (e4m3 values, e8m0 scale per 32 along k).

    contract_variant 2 = block-scaled tcgen05 contraction; 0 = expand the operands to bf16
    (exactly) and run the bf16 contraction: the cross-check of variant 2.
    """
    n = z.shape[0]
    st = stream()
    pitch8 = _round_up(n, 16)
    stride8 = n * pitch8
    a8, b8 = ws.buf[3].view(torch.uint8), ws.buf[4].view(torch.uint8)
    sa, sb = ws.mx_scales()
    x = ws.buf[2]
    call("b200pf_trimul_producer_mx", ptr(z), ptr(mask_u8), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]),
         ptr(a8), ptr(b8), ptr(sa), ptr(sb), stride8, pitch8, n, n, int(incoming), st)
    if contract_variant == 2:
        pa = Planes(ptr(a8), stride8, 0, pitch8, n, n, 1, 0)
        pb = Planes(ptr(b8), stride8, 0, pitch8, n, n, 1, 0)
        call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), ptr(sa), ptr(sb), ptr(x), ws.plane_stride, ws.pitch, 0, 0, C_Z, 2, st)
    else:
        a, b = ws.buf[0], ws.buf[1]
        for src, sc, dst in ((a8, sa, a), (b8, sb, b)):
            call("b200pf_mx_dequant", ptr(src), ptr(sc), ptr(dst), stride8, pitch8, ws.plane_stride, ws.pitch, n, n, C_Z, st)
        pa = Planes(ptr(a), ws.plane_stride, 0, ws.pitch, n, n, 1, 0)
        pb = Planes(ptr(b), ws.plane_stride, 0, ws.pitch, n, n, 1, 0)
        call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), ws.plane_stride, ws.pitch,
             0, 0, C_Z, 0, st)
    if before_z_write is not None:
        before_z_write()
    trimul_epilogue(z, x, ws.plane_stride, ws.pitch, w, n, n)


def tri_att_bf16(z: torch.Tensor, masks: PairMasks, w: Dict[str, torch.Tensor], ws: Workspace, ending: bool) -> None:
    n = z.shape[0]
    q, k, v, g, o = ws.buf
    st = stream()
    bias_hs, bias_qs = ws.pitch, 4 * ws.pitch          # layout [query][head][key]: a row shard is contiguous
    call("b200pf_triatt_producer", ptr(z), *triatt_producer_weights(w), ptr(q), ptr(k), ptr(v), ptr(g),
         ptr(ws.tri_bias), bias_hs, bias_qs, ws.pitch, n, n, int(ending), st)
    if ending:      # line = column j: o element (line, pos) -> z position [pos][line]
        o_ls, o_ps = C_Z, n * C_Z
    else:
        o_ls, o_ps = n * C_Z, C_Z
    lines_mask = masks.cols if ending else masks.rows
    call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), ws.pitch, ptr(ws.tri_bias), bias_hs, bias_qs,
         ptr(lines_mask), masks.pitch, ptr(o), o_ls, o_ps, n, n, st)
    call("b200pf_triatt_epilogue", ptr(z), ptr(o), ptr(g), ptr(w["w_o"]), n * n, st)


def transition_z_bf16(z: torch.Tensor, w: Dict[str, torch.Tensor]) -> None:
    rows = z.shape[0] * z.shape[1]
    call("b200pf_transition_z_tc", ptr(z), ptr(w["ln_gamma"]), ptr(w["ln_beta"]), ptr(w["w12_tc"]), ptr(w["w3"]), rows, stream())


# ------------------------------------------------------------------------------------------------
# fp32 tier (un-fused SIMT kernels) - also the single-track path of every tier
# ------------------------------------------------------------------------------------------------
def _empty(rows: int, c: int, like: torch.Tensor) -> torch.Tensor:
    return torch.empty(rows, c, dtype=torch.float32, device=like.device)


def f32_layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    rows, c = x.numel() // x.shape[-1], x.shape[-1]
    y = _empty(rows, c, x)
    call("b200pf_f32_layernorm", ptr(x), ptr(gamma), ptr(beta), ptr(y), rows, c, stream())
    return y


def f32_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    k = w.shape[1]
    rows = x.numel() // k
    if out is None:
        out = _empty(rows, w.shape[0], x)
    call("b200pf_f32_linear", ptr(x), ptr(w), ptr(bias), ptr(out), rows, k, w.shape[0], int(accumulate), stream())
    return out


def f32_gate(a: torch.Tensor, b: torch.Tensor, mode: int, row_mask: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    c = a.shape[-1]
    rows = a.numel() // c
    if out is None:
        out = _empty(rows, c, a)
    call("b200pf_f32_gate", ptr(a), ptr(b), ptr(row_mask), ptr(out), rows, c, mode, stream())
    return out


def tri_mul_f32(z: torch.Tensor, mask_u8: torch.Tensor, w: Dict[str, torch.Tensor], incoming: bool) -> None:
    n = z.shape[0]
    x = f32_layernorm(z, w["norm_in.weight"], w["norm_in.bias"])
    u = f32_gate(f32_linear(x, w["p_in.weight"]), f32_linear(x, w["g_in.weight"]), 0, mask_u8)     # [N*N, 2D]
    d = u.shape[1] // 2
    t = _empty(n * n, d, z)
    call("b200pf_f32_trimul_contract", ptr(u), u.data_ptr() + 4 * d, ptr(t), n, d, 2 * d, int(incoming), stream())
    tn = f32_layernorm(t, w["norm_out.weight"], w["norm_out.bias"])
    f32_gate(f32_linear(tn, w["p_out.weight"]), f32_linear(x, w["g_out.weight"]), 2, out=z)


def _attention_f32(q, k, v, bias, bias_strides, mask_u8, mask_strides, batch, n_q, n_k, heads, hd, rs, ps,
                   scale, inf_value, order) -> torch.Tensor:
    o = torch.empty_like(q)
    call("b200pf_f32_attention", ptr(q), ptr(k), ptr(v), ptr(o), ptr(bias), *bias_strides, ptr(mask_u8),
         *mask_strides, batch, n_q, n_k, heads, hd, rs, ps, scale, inf_value, order, stream())
    return o


def tri_att_f32(z: torch.Tensor, mask_u8: torch.Tensor, w: Dict[str, torch.Tensor], ending: bool) -> None:
    n, c = z.shape[0], z.shape[-1]
    st = stream()
    if ending:      # the reference transposes z and the mask, runs the starting-node path, transposes back
        src = torch.empty_like(z)
        call("b200pf_f32_transpose01", ptr(z), ptr(src), n, c, 0, st)
        mask_ls, mask_ks = 1, n
    else:
        src = z
        mask_ls, mask_ks = n, 1
    heads = w["linear.weight"].shape[0]
    hd = w["mha.linear_q.weight"].shape[0] // heads
    x = f32_layernorm(src, w["layer_norm.weight"], w["layer_norm.bias"])
    bias = torch.empty(heads, n * n, dtype=torch.float32, device=z.device)
    if c == C_Z and heads in (4, 16):       # one fused pass over z
        call("b200pf_ln_proj_heads", ptr(src), ptr(w["layer_norm.weight"]), ptr(w["layer_norm.bias"]),
             ptr(w["linear.weight"]), ptr(bias), n * n, n * n, c, heads, st)
    else:                                   # other widths / head counts: the normalised rows through the transposing linear
        call("b200pf_f32_linear_t", ptr(x), ptr(w["linear.weight"]), None, ptr(bias), n * n, n * n, c, heads, st)
    q = f32_linear(x, w["mha.linear_q.weight"])
    k = f32_linear(x, w["mha.linear_k.weight"])
    v = f32_linear(x, w["mha.linear_v.weight"])
    g = f32_linear(x, w["mha.linear_g.weight"])
    o = _attention_f32(q, k, v, bias, (n * n, n, 1), mask_u8, (mask_ls, mask_ks), n, n, n, heads, hd,
                       n * heads * hd, heads * hd, 1.0 / math.sqrt(hd), 1e9, 0)
    og = f32_gate(o, g, 0)
    if ending:
        upd = f32_linear(og, w["mha.linear_o.weight"])
        call("b200pf_f32_transpose01", ptr(upd), ptr(z), n, c, 1, st)
    else:
        f32_linear(og, w["mha.linear_o.weight"], out=z, accumulate=True)


def transition_f32(x_res: torch.Tensor, w: Dict[str, torch.Tensor]) -> None:
    x = f32_layernorm(x_res, w["norm.weight"], w["norm.bias"])
    h = f32_gate(f32_linear(x, w["fc1.weight"]), f32_linear(x, w["fc2.weight"]), 1)
    f32_linear(h, w["fc3.weight"], out=x_res, accumulate=True)


def pair_bias_heads(z: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    """bias[h][i_local*N + j] of the single-track attention: one fp32 pass over the (local rows of) z."""
    rows, c = z.shape[0] * z.shape[1], z.shape[-1]          # z may be a row shard [nr, N, c_z]
    heads = w["proj_z.1.weight"].shape[0]
    bias = torch.empty(heads, rows, dtype=torch.float32, device=z.device)
    if c == C_Z and heads in (4, 16):
        call("b200pf_ln_proj_heads", ptr(z), ptr(w["proj_z.0.weight"]), ptr(w["proj_z.0.bias"]),
             ptr(w["proj_z.1.weight"]), ptr(bias), rows, rows, c, heads, stream())
    else:
        x = f32_layernorm(z, w["proj_z.0.weight"], w["proj_z.0.bias"])
        call("b200pf_f32_linear_t", ptr(x), ptr(w["proj_z.1.weight"]), None, ptr(bias), rows, rows, c, heads, stream())
    return bias


def pack_single_track(w_att: Dict[str, torch.Tensor], w_trans: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Concatenated fp32 weights so that q|g, k|v and fc1|fc2 are one GEMM launch each."""
    cs = w_att["proj_q.weight"].shape[0]
    return {
        "w_qg": torch.cat([w_att["proj_q.weight"], w_att["proj_g.weight"]], 0).contiguous(),
        "b_qg": torch.cat([w_att["proj_q.bias"], torch.zeros(cs, device=w_att["proj_q.bias"].device)], 0).contiguous(),
        "w_kv": torch.cat([w_att["proj_k.weight"], w_att["proj_v.weight"]], 0).contiguous(),
        "w_12": torch.cat([w_trans["fc1.weight"], w_trans["fc2.weight"]], 0).contiguous(),
    }


def single_track_local(s: torch.Tensor, z_rows: torch.Tensor, tok_mask_u8: torch.Tensor, w_norm: Dict[str, torch.Tensor],
                       w_att: Dict[str, torch.Tensor], fused: Dict[str, torch.Tensor], num_heads: int,
                       r0: int = 0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated attention output sigmoid(g) * softmax(...) v for the query rows [r0, r0 + z_rows.shape[0]) (fp32).
    ``bias`` = pair_bias_heads(z_rows, w_att) when the caller has computed it already (then z_rows is only read
    for its shape)."""
    n, cs = s.shape
    nq = z_rows.shape[0]
    hd = cs // num_heads
    st = stream()
    sn = f32_layernorm(s, w_norm["weight"], w_norm["bias"])
    qg = f32_linear(sn[r0:r0 + nq], fused["w_qg"], fused["b_qg"])                       # [nq, 2 cs]: q | g
    pitch = _round_up(n, 4)
    kvt = torch.empty(2 * cs, pitch, dtype=torch.float32, device=s.device)              # [k rows | v rows][key]
    call("b200pf_f32_linear_t", ptr(sn), ptr(fused["w_kv"]), None, ptr(kvt), pitch, n, cs, 2 * cs, st)
    if bias is None:
        bias = pair_bias_heads(z_rows, w_att)                                            # [heads][nq * n]
    o = torch.empty(nq, cs, dtype=torch.float32, device=s.device)
    call("b200pf_f32_sattention", ptr(qg), 2 * cs, qg.data_ptr() + 4 * cs, 2 * cs, ptr(kvt), kvt.data_ptr() + 4 * cs * pitch, pitch,
         ptr(o), cs, ptr(bias), nq * n, n, ptr(tok_mask_u8), nq, n, num_heads, hd, 1.0 / math.sqrt(hd), 1e6, st)
    return o


def single_track_finish(s: torch.Tensor, og_all: torch.Tensor, w_att: Dict[str, torch.Tensor],
                        w_trans: Dict[str, torch.Tensor], fused: Dict[str, torch.Tensor]) -> None:
    """s += proj_o(gated attention output); s += Transition(s) (tt_bio/reference.py:906-911)."""
    n, cs = s.shape
    f32_linear(og_all, w_att["proj_o.weight"], out=s, accumulate=True)
    x = f32_layernorm(s, w_trans["norm.weight"], w_trans["norm.bias"])
    h12 = f32_linear(x, fused["w_12"])                                                  # [n, 8 cs]: fc1 | fc2
    hidden = h12.shape[1] // 2
    h = torch.empty(n, hidden, dtype=torch.float32, device=s.device)
    call("b200pf_f32_gate_strided", ptr(h12), 2 * hidden, h12.data_ptr() + 4 * hidden, 2 * hidden, ptr(h), hidden,
         n, hidden, 1, stream())
    f32_linear(h, w_trans["fc3.weight"], out=s, accumulate=True)


def single_track(s: torch.Tensor, z: torch.Tensor, tok_mask_u8: torch.Tensor, w_norm: Dict[str, torch.Tensor],
                 w_att: Dict[str, torch.Tensor], w_trans: Dict[str, torch.Tensor], num_heads: int,
                 fused: Optional[Dict[str, torch.Tensor]] = None, after_z_read=None) -> None:
    """s += AttentionPairBias(LN(s), z); s += Transition(s) in fp32 (tt_bio/reference.py:906-912).
    The pair-bias projection, the single track's only read of z, comes first; ``after_z_read`` is called behind it."""
    if fused is None:
        fused = pack_single_track(w_att, w_trans)
    bias = pair_bias_heads(z, w_att)
    if after_z_read is not None:
        after_z_read()
    og = single_track_local(s, z, tok_mask_u8, w_norm, w_att, fused, num_heads, 0, bias)
    single_track_finish(s, og, w_att, w_trans, fused)
