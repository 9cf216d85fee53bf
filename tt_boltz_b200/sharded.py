"""Row-sharded Pairformer trunk for one large complex on the GPUs of one box.

One process per GPU (``torch.distributed``, backend NCCL over NVLink / NVSwitch).  Rank r owns
rows R_r = [r*nr, (r+1)*nr) of the fp32 pair tensor, nr = N / P; the single representation s is
replicated.  Exchanges per block (everything else is row-local):

  tri_mul_out    all-gather of the k-side operand b (bf16 planes)
  tri_mul_in     all-to-all of a^T blocks (destination = owner of the output rows) and
                 all-gather of b^T; the contraction index arrives split in P segments
  tri_att_start  all-gather of the triangle bias [query][head][key] (8 MiB at N = 1024)
  tri_att_end    all-to-all row shard -> column shard of z (fp32), bias all-gather, and the
                 all-to-all back of the updated column shard
  single track   all-gather of the gated attention output of the local query rows

The plumbing helpers below work on CPU tensors with the gloo backend as well, which is how the
partition / index logic is tested without GPUs.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from . import ops, weights
from ._lib import PlaneOut, Planes, call, ptr, stream
from .pairformer import B200PairformerLayer, _mask_u8

C_Z = 128


# ------------------------------------------------------------------------------------------------
# plumbing (backend-agnostic)
# ------------------------------------------------------------------------------------------------
def all_gather_cat(x: torch.Tensor, group=None) -> torch.Tensor:
    """[P, *x.shape]: slot s holds rank s's tensor."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)      # one NCCL call, no staging copies
    else:
        dist.all_gather(list(out.unbind(0)), x.contiguous(), group=group)
    return out


def all_to_all_blocks(send: torch.Tensor, group=None) -> torch.Tensor:
    """send[t] goes to rank t; recv[s] is what rank s sent to this rank."""
    send = send.contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def rows_to_cols(z_loc: torch.Tensor, group=None) -> torch.Tensor:
    """Row shard [nr, N, C] -> column shard stored [N, nr, C] (element [i][j_local])."""
    world = dist.get_world_size(group)
    nr, n, c = z_loc.shape
    send = z_loc.view(nr, world, nr, c).permute(1, 0, 2, 3)      # [dest t][i_local][j_local][c]
    return all_to_all_blocks(send, group).view(n, nr, c)         # [src s * nr + i_local][j_local][c]


def cols_to_rows(zc: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of rows_to_cols: column shard [N, nr, C] -> row shard [nr, N, C]."""
    world = dist.get_world_size(group)
    n, nr, c = zc.shape
    recv = all_to_all_blocks(zc.view(world, nr, nr, c), group)   # recv[s] = rows R_r, cols R_s
    return recv.permute(1, 0, 2, 3).reshape(nr, n, c).contiguous()


def shard_rows(n: int, rank: int, world: int) -> Tuple[int, int]:
    if n % world:
        raise RuntimeError(f"row sharding needs N divisible by the number of ranks (N={n}, P={world})")
    nr = n // world
    return rank * nr, nr


# ------------------------------------------------------------------------------------------------
# one sharded block on the GPU
# ------------------------------------------------------------------------------------------------
def _ru8(x: int) -> int:
    return (x + 7) // 8 * 8


def _bf16(n_elems: int, dev) -> torch.Tensor:
    return torch.empty(n_elems, dtype=torch.bfloat16, device=dev)


def sharded_block(layer: B200PairformerLayer, s: Optional[torch.Tensor], z_loc: torch.Tensor,
                  tok_mask_u8: Optional[torch.Tensor], masks: ops.PairMasks, rank: int, world: int,
                  group=None) -> torch.Tensor:
    """Update the local row shard z_loc [nr, N, 128] (returned; may be a new tensor) and s in place."""
    pk = layer._pack(z_loc.device)
    dev = z_loc.device
    nr, n, _ = z_loc.shape
    r0 = rank * nr
    if nr % 128:
        raise RuntimeError("the sharded bf16 path needs N / P to be a multiple of 128 tokens")
    pn, pr = _ru8(n), _ru8(nr)
    st = stream()
    mask_loc = masks.pm[r0:r0 + nr]

    # ---- triangle multiplication, outgoing -------------------------------------------------------
    w = pk["tri_mul_out"]
    a_loc, b_loc, x = _bf16(C_Z * nr * pn, dev), _bf16(C_Z * nr * pn, dev), _bf16(C_Z * nr * pn, dev)
    oa, ob = PlaneOut(ptr(a_loc), nr * pn, 0, 0), PlaneOut(ptr(b_loc), nr * pn, 0, 0)
    call("b200pf_trimul_producer", ptr(z_loc), ptr(mask_loc), *ops.trimul_producer_weights(w, layer.row_impl),
         C.byref(oa), C.byref(ob), pn, nr, n, 0, 0, layer.row_impl, st)
    b_all = all_gather_cat(b_loc, group)                                             # [P][D][nr][pn]
    pa = Planes(ptr(a_loc), nr * pn, 0, pn, nr, n, 1, 0)
    pb = Planes(ptr(b_all), nr * pn, C_Z * nr * pn, pn, nr, n, world, 0)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), nr * pn, pn, C_Z, layer.contract_variant, st)
    ops.trimul_epilogue(z_loc, x, nr * pn, pn, w, nr, n, layer.row_impl)

    # ---- triangle multiplication, incoming -------------------------------------------------------
    w = pk["tri_mul_in"]
    at_send = _bf16(world * C_Z * nr * pr, dev)                                      # [dest][D][i_local][k_local]
    bt_loc = _bf16(C_Z * n * pr, dev)                                                # [D][j][k_local]
    oa = PlaneOut(ptr(at_send), nr * pr, C_Z * nr * pr, nr)
    ob = PlaneOut(ptr(bt_loc), n * pr, 0, 0)
    call("b200pf_trimul_producer", ptr(z_loc), ptr(mask_loc), *ops.trimul_producer_weights(w, layer.row_impl),
         C.byref(oa), C.byref(ob), pr, nr, n, 1, 0, layer.row_impl, st)
    at_recv = all_to_all_blocks(at_send.view(world, -1), group)                      # [src][D][i_local][k_local of src]
    bt_all = all_gather_cat(bt_loc, group)                                           # [src][D][j][k_local of src]
    pa = Planes(ptr(at_recv), nr * pr, C_Z * nr * pr, pr, nr, nr, world, 1)
    pb = Planes(ptr(bt_all), n * pr, C_Z * n * pr, pr, n, nr, world, 1)
    call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), None, None, ptr(x), nr * pn, pn, C_Z, layer.contract_variant, st)
    ops.trimul_epilogue(z_loc, x, nr * pn, pn, w, nr, n, layer.row_impl)
    del a_loc, b_loc, b_all, at_send, at_recv, bt_loc, bt_all, x

    # ---- triangle attention, starting node (lines = local rows) ---------------------------------
    w = pk["tri_att_start"]
    q, k, v, g, o = (_bf16(nr * n * C_Z, dev) for _ in range(5))
    bias_loc = _bf16(nr * 4 * pn, dev)
    call("b200pf_triatt_producer", ptr(z_loc), *ops.triatt_producer_weights(w, layer.row_impl), ptr(q), ptr(k), ptr(v), ptr(g),
         ptr(bias_loc), pn, 4 * pn, pn, nr, n, 0, layer.row_impl, st)
    bias_all = all_gather_cat(bias_loc, group)                                       # [query][head][key]
    call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), pn, ptr(bias_all), pn, 4 * pn, ptr(masks.rows[r0:r0 + nr]),
         masks.pitch, ptr(o), n * C_Z, C_Z, nr, n, st)
    call("b200pf_triatt_epilogue", ptr(z_loc), ptr(o), ptr(g), ptr(w["w_o"]), nr * n, st)

    # ---- triangle attention, ending node (lines = local columns of the column shard) ------------
    w = pk["tri_att_end"]
    zc = rows_to_cols(z_loc, group)                                                  # [N][nr][128] fp32
    call("b200pf_triatt_producer", ptr(zc), *ops.triatt_producer_weights(w, layer.row_impl), ptr(q), ptr(k), ptr(v), ptr(g),
         ptr(bias_loc), pn, 4 * pn, pn, n, nr, 1, layer.row_impl, st)
    bias_all = all_gather_cat(bias_loc, group)
    call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), pn, ptr(bias_all), pn, 4 * pn, ptr(masks.cols[r0:r0 + nr]),
         masks.pitch, ptr(o), C_Z, nr * C_Z, nr, n, st)
    call("b200pf_triatt_epilogue", ptr(zc), ptr(o), ptr(g), ptr(w["w_o"]), n * nr, st)
    z_loc = cols_to_rows(zc, group)
    del q, k, v, g, o, zc, bias_loc, bias_all

    # ---- pair transition ---------------------------------------------------------------------------
    ops.transition_z_bf16(z_loc, pk["transition_z"], layer.row_impl)

    # ---- single track: attention for the local query rows, the rest replicated --------------------
    if layer.with_s and s is not None:
        og_loc = ops.single_track_local(s, z_loc, tok_mask_u8, pk["pre_norm_s"], pk["attention"], pk["s_fused"],
                                        layer.num_heads, r0)
        og_all = all_gather_cat(og_loc, group).view(n, s.shape[1])
        ops.single_track_finish(s, og_all, pk["attention"], pk["transition_s"], pk["s_fused"])
    return z_loc


class ShardedPairformerModule(nn.Module):
    """Same constructor and forward signature as ``B200PairformerModule``; every rank passes the
    full (replicated) inputs and receives the full outputs, the blocks run row-sharded in between."""

    def __init__(self, token_s: int, token_z: int, num_blocks: int, num_heads: int = 16, dropout: float = 0.25,
                 pairwise_head_width: int = 32, pairwise_num_heads: int = 4, post_layer_norm: bool = False,
                 activation_checkpointing: bool = False, v2: bool = False, precision: str = "bf16", group=None,
                 **kwargs) -> None:
        super().__init__()
        if precision != "bf16":
            raise NotImplementedError("the sharded trunk is built for the bf16 tier")
        self.group = group
        self.layers = nn.ModuleList([
            B200PairformerLayer(token_s, token_z, num_heads, dropout, pairwise_head_width, pairwise_num_heads,
                                post_layer_norm, v2, precision, with_s=True) for _ in range(num_blocks)])

    def forward_sharded(self, s: torch.Tensor, z_loc: torch.Tensor, mask: Optional[torch.Tensor],
                        pair_mask: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """z_loc [nr, N, 128] fp32 row shard in, row shard out (no gather): the resident-trunk form."""
        rank, world = dist.get_rank(self.group), dist.get_world_size(self.group)
        n = z_loc.shape[1]
        with torch.cuda.device(z_loc.device), torch.no_grad():
            pm = ops.PairMasks(_mask_u8(pair_mask, (n, n), z_loc.device))
            tm = _mask_u8(mask, (n,), z_loc.device)
            sw = s.to(torch.float32).clone()
            for layer in self.layers:
                z_loc = sharded_block(layer, sw, z_loc, tm, pm, rank, world, self.group)
        return sw, z_loc

    def forward(self, s: torch.Tensor, z: torch.Tensor, mask: Optional[torch.Tensor] = None,
                pair_mask: Optional[torch.Tensor] = None, use_kernels: bool = False
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        if not z.is_cuda:
            raise RuntimeError("ShardedPairformerModule: inputs must be CUDA tensors (there is no CPU path)")
        rank, world = dist.get_rank(self.group), dist.get_world_size(self.group)
        n = z.shape[1]
        r0, nr = shard_rows(n, rank, world)
        z_loc = z[0, r0:r0 + nr].to(torch.float32).clone(memory_format=torch.contiguous_format)
        sw, z_loc = self.forward_sharded(s[0], z_loc, mask, pair_mask)
        z_out = all_gather_cat(z_loc, self.group).view(1, n, n, z.shape[-1])
        return sw.unsqueeze(0).to(s.dtype), z_out.to(z.dtype)
