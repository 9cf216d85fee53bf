"""Row-sharded Pairformer trunk for one large complex on the GPUs of one box.

One process per GPU (``torch.distributed``, backend NCCL over NVLink / NVSwitch).  Rank r owns
rows R_r = [r*nr, (r+1)*nr) of the fp32 pair tensor, nr = N / P; the single representation s is
replicated.  Exchanges per block (everything else is row-local):

  tri_mul_out/in all-to-all of the a and b planes from row shards to CHANNEL shards (each rank
                 contracts 128/P channels for all rows; the operands arrive split in P row
                 segments (outgoing) or P segments of the contraction index (incoming)), and the
                 all-to-all of the result back to row shards
  tri_att_start  all-gather of the triangle bias [query][head][key] (8 MiB at N = 1024)
  tri_att_end    all-to-all row shard -> column shard of z (fp32), bias all-gather, and the
                 all-to-all back of the updated column shard
  single track   attention, output projection and transition for the local rows, all-gather of s

The plumbing helpers below work on CPU tensors with the gloo backend as well, which is how the
partition / index logic is tested without GPUs.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from . import ops, weights
from ._lib import PeerSync, PlaneOut, Planes, call, device_status, ptr, stream
from .pairformer import B200PairformerLayer, SideTrack, _mask_u8

C_Z = 128


# ------------------------------------------------------------------------------------------------
# plumbing (backend-agnostic)
# ------------------------------------------------------------------------------------------------
def all_gather_cat(x: torch.Tensor, group=None, tag: Optional[str] = None, channel: int = 0) -> torch.Tensor:
    """[P, *x.shape]: slot s holds rank s's tensor.  With a ``tag`` on CUDA: peer writes (see all_to_all_blocks);
    ``channel`` names the barrier state of the stream the call is enqueued on (see peer_barrier)."""
    world = dist.get_world_size(group)
    x = x.contiguous()
    nbytes = x.numel() * x.element_size()
    if x.is_cuda and tag is not None and _PEER_COPY["enabled"] and nbytes % 16 == 0:
        peer = _peer_buffers(tag, world * x.numel(), x.dtype, x.device, group)
        if peer is not None:
            recv, hdl, ptrs = peer
            call("b200pf_peer_broadcast_sync", ptr(x), ptrs, nbytes, dist.get_rank(group), world,
                 C.byref(_next_sync(x.device, group, channel)), stream())
            return recv.view((world,) + tuple(x.shape))
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x, group=group)      # one NCCL call, no staging copies
    else:
        dist.all_gather(list(out.unbind(0)), x, group=group)
    return out


# The receive buffers are plain peer mappings; nothing here uses NVLink multicast, so the allocator is told
# not to bind a multicast object to them (a rank that dies while bound can fault its peers' links).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

# Symmetric (peer-mapped) receive buffers of the peer-write all-to-all: two per call site and size, used in turn.
_SYMM: Dict[tuple, tuple] = {}
_SYMM_TURN: Dict[tuple, int] = {}
_PEER_COPY = {"enabled": os.environ.get("B200PF_PEER_COPY", "1") != "0"}       # "0": every exchange through NCCL
# A rank that never arrives ends the wait after this long: the barrier kernel sets bit 4 of the device status word
# and returns (no trap, the context stays usable); ShardedPairformerModule.forward reads the word and raises.
_BARRIER_TIMEOUT_MS = int(os.environ.get("B200PF_BARRIER_TIMEOUT_MS", "20000"))
_BARRIERS: Dict[tuple, list] = {}


def _barrier_state(device: torch.device, group, channel: int) -> list:
    """[pad, handle, pad pointers, generation] of one barrier channel: a small symmetric allocation per (device,
    group, channel), zeroed before the first use.  The generation counter lives on the host and grows by one per
    barrier, the same on every rank because every rank enqueues the same sequence of exchanges ON ONE STREAM.
    Exchanges enqueued on another stream (the single track's side stream) may interleave differently with them on
    different ranks, so they use a channel, i.e. pads and a counter, of their own."""
    key = (device.index, id(group), channel)
    st = _BARRIERS.get(key)
    if st is None:
        import torch.distributed._symmetric_memory as symm
        pg = group if group is not None else dist.group.WORLD
        pad = symm.empty(64, dtype=torch.int32, device=device)
        pad.zero_()
        hdl = symm.rendezvous(pad, pg)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                      # every pad is zero before any rank signals
        ptrs = (C.c_ulonglong * hdl.world_size)(*[int(p) for p in hdl.buffer_ptrs])
        st = _BARRIERS[key] = [pad, hdl, ptrs, 0]
    return st


def _next_sync(device: torch.device, group, channel: int) -> PeerSync:
    """The barrier description for the next exchange of this channel (``b200pf_peer_*_sync``)."""
    st = _barrier_state(device, group, channel)
    st[3] = (st[3] + 1) & 0xFFFFFFFF
    return PeerSync(st[2], st[3], _BARRIER_TIMEOUT_MS * 1000000, channel)


def peer_barrier(device: torch.device, group=None, channel: int = 0) -> None:
    """Enqueue the library's own cross-rank barrier alone (``b200pf_peer_barrier``) on the current stream."""
    st = _barrier_state(device, group, channel)
    st[3] = (st[3] + 1) & 0xFFFFFFFF
    call("b200pf_peer_barrier", st[2], st[3], dist.get_rank(group), dist.get_world_size(group),
         _BARRIER_TIMEOUT_MS * 1000000, stream())


def _symm_buffer(tag: str, numel: int, dtype: torch.dtype, device: torch.device, group):
    key = (tag, numel, dtype, device.index)
    turn = _SYMM_TURN.get(key, 0)
    _SYMM_TURN[key] = turn ^ 1
    key = key + (turn,)
    if key not in _SYMM:
        import torch.distributed._symmetric_memory as symm
        buf = symm.empty(numel, dtype=dtype, device=device)
        hdl = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
        ptrs = (C.c_ulonglong * hdl.world_size)(*[int(p) for p in hdl.buffer_ptrs])
        _SYMM[key] = (buf, hdl, ptrs)
    return _SYMM[key]


def _peer_buffers(tag: str, numel: int, dtype: torch.dtype, device: torch.device, group):
    """Receive buffer, handle and peer pointers, or None when symmetric memory cannot be set up on this system
    (the allocation and the rendezvous are collective, so every rank takes the same branch): the exchange then
    goes through NCCL for the rest of the process."""
    try:
        return _symm_buffer(tag, numel, dtype, device, group)
    except (RuntimeError, ImportError, AttributeError) as exc:        # no peer mapping / API missing in this torch
        if _PEER_COPY["enabled"]:
            _PEER_COPY["enabled"] = False
            if dist.get_rank(group) == 0:
                print(f"b200pf: symmetric memory unavailable ({exc}); exchanges go through NCCL", flush=True)
        return None


def all_to_all_blocks(send: torch.Tensor, group=None, tag: Optional[str] = None, barrier: bool = True) -> torch.Tensor:
    """send[t] goes to rank t; recv[s] is what rank s sent to this rank.

    On CUDA with a ``tag`` (one per call site) every rank writes its blocks straight into the destination
    ranks' symmetric receive buffers over NVLink with one kernel (``b200pf_peer_scatter``), followed by one
    device-side barrier at the end of the same kernel that says every block has landed (``barrier=False`` leaves it
    to a following exchange of the same group of calls).  Each call site alternates between two receive
    buffers: a rank can only pass the barrier of exchange k+1 after every rank has enqueued it, i.e. after
    their consumers of exchange k in stream order, so exchange k+2 may overwrite buffer k without another
    barrier.  The returned tensor is the receive buffer: valid until the second-next exchange of the same
    tag and size.  Otherwise (CPU / gloo, no tag, or B200PF_PEER_COPY=0) it is ``all_to_all_single``.
    """
    send = send.contiguous()
    if send.is_cuda and tag is not None and _PEER_COPY["enabled"]:
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        peer = _peer_buffers(tag, send.numel(), send.dtype, send.device, group)
        if peer is not None:
            recv, hdl, ptrs = peer
            nbytes = send.numel() * send.element_size() // world
            if barrier:
                call("b200pf_peer_scatter_sync", ptr(send), ptrs, nbytes, rank, world, C.byref(_next_sync(send.device, group, 0)), stream())
            else:       # the caller follows up with another exchange that carries the barrier for both
                call("b200pf_peer_scatter", ptr(send), ptrs, nbytes, rank, world, stream())
            return recv.view(send.shape)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def _strided_exchange(tag: str, src: torch.Tensor, out_numel: int, chunk_elems: int, chunks: int, src_block: int, src_chunk: int,
                      dst_slot: int, dst_chunk: int, group):
    """One launch of b200pf_peer_scatter_strided_sync (strides in ELEMENTS of src; the barrier is the kernel's tail)
    into the symmetric receive buffer of ``tag``; None when peer copies are off or unavailable."""
    if not (src.is_cuda and _PEER_COPY["enabled"]):
        return None
    peer = _peer_buffers(tag, out_numel, src.dtype, src.device, group)
    if peer is None:
        return None
    recv, _, ptrs = peer
    e = src.element_size()
    call("b200pf_peer_scatter_strided_sync", ptr(src), ptrs, chunk_elems * e, chunks, src_block * e, src_chunk * e, dst_slot * e, dst_chunk * e,
         dist.get_rank(group), dist.get_world_size(group), C.byref(_next_sync(src.device, group, 0)), stream())
    return recv


def rows_to_cols(z_loc: torch.Tensor, group=None) -> torch.Tensor:
    """Row shard [nr, N, C] -> column shard stored [N, nr, C] (element [i][j_local]).  On CUDA the pieces are read
    out of the row shard and written into the receivers' column shards directly (no packing copy); the result is
    then the receive buffer (valid until the second-next call)."""
    world = dist.get_world_size(group)
    nr, n, c = z_loc.shape
    # block for rank t = my rows x its columns: nr pieces (one per local row) of nr*c contiguous elements
    recv = _strided_exchange("z_rows_to_cols", z_loc.contiguous(), n * nr * c, nr * c, nr, nr * c, n * c, nr * nr * c, nr * c, group)
    if recv is not None:
        return recv.view(n, nr, c)
    send = z_loc.view(nr, world, nr, c).permute(1, 0, 2, 3)      # [dest t][i_local][j_local][c]
    return all_to_all_blocks(send, group, "z_rows_to_cols").view(n, nr, c)   # [src s * nr + i_local][j_local][c]


# Around the sharded ending-node attention z crosses the wire in bf16 and only the update comes back (half the bytes
# of the fp32 round trip); "0" keeps the fp32 exchange, which reproduces the one-GPU result bit for bit.
_BF16_EXCHANGE = {"enabled": os.environ.get("B200PF_BF16_EXCHANGE", "1") != "0"}


def rows_to_cols_bf16(z_loc: torch.Tensor, group=None) -> Optional[torch.Tensor]:
    """fp32 row shard [nr, N, C] -> bf16 column shard [N, nr, C], narrowed by the exchange kernel itself; None when
    peer copies are off or unavailable (the caller then takes the fp32 path)."""
    if not (z_loc.is_cuda and _PEER_COPY["enabled"] and z_loc.dtype == torch.float32):
        return None
    nr, n, c = z_loc.shape
    peer = _peer_buffers("z_rows_to_cols_bf16", n * nr * c, torch.bfloat16, z_loc.device, group)
    if peer is None:
        return None
    recv, _, ptrs = peer
    call("b200pf_peer_scatter_strided_f32_bf16_sync", ptr(z_loc), ptrs, nr * c, nr, nr * c, n * c, nr * nr * c, nr * c,
         dist.get_rank(group), dist.get_world_size(group), C.byref(_next_sync(z_loc.device, group, 0)), stream())
    return recv.view(n, nr, c)


def cols_to_rows(zc: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of rows_to_cols: column shard [N, nr, C] -> row shard [nr, N, C].  On CUDA every piece lands at its
    place in the receiver's row shard (no unpacking copy); the result is then the receive buffer (valid until the
    second-next call)."""
    world = dist.get_world_size(group)
    n, nr, c = zc.shape
    # block for rank t = its rows x my columns: piece i_local goes to row i_local, columns [rank*nr, (rank+1)*nr)
    recv = _strided_exchange("z_cols_to_rows", zc.contiguous(), nr * n * c, nr * c, nr, nr * nr * c, nr * c, nr * c, n * c, group)
    if recv is not None:
        return recv.view(nr, n, c)
    recv = all_to_all_blocks(zc.view(world, nr, nr, c), group, "z_cols_to_rows")   # recv[s] = rows R_r, cols R_s
    return recv.permute(1, 0, 2, 3).reshape(nr, n, c).contiguous()


def shard_rows(n: int, rank: int, world: int) -> Tuple[int, int]:
    if n % world:
        raise RuntimeError(f"row sharding needs N divisible by the number of ranks (N={n}, P={world})")
    nr = n // world
    return rank * nr, nr


# ------------------------------------------------------------------------------------------------
# one sharded block on the GPU
# ------------------------------------------------------------------------------------------------
def _lib_handle():
    from . import _lib
    return _lib.load()


def _ru8(x: int) -> int:
    return (x + 7) // 8 * 8


def _bf16(n_elems: int, dev) -> torch.Tensor:
    return torch.empty(n_elems, dtype=torch.bfloat16, device=dev)


def sharded_block(layer: B200PairformerLayer, s: Optional[torch.Tensor], z_loc: torch.Tensor,
                  tok_mask_u8: Optional[torch.Tensor], masks: ops.PairMasks, rank: int, world: int,
                  group=None, side: Optional[SideTrack] = None) -> torch.Tensor:
    """Update the local row shard z_loc [nr, N, 128] (returned; may be a new tensor) and s in place.  With a
    ``side`` track the update of s is only enqueued on its stream: the caller joins it before reading s."""
    pk = layer._pack(z_loc.device)
    dev = z_loc.device
    nr, n, _ = z_loc.shape
    r0 = rank * nr
    if nr % 128:
        raise RuntimeError("the sharded bf16 path needs N / P to be a multiple of 128 tokens")
    pn, pr = _ru8(n), _ru8(nr)
    st = stream()
    mask_loc = masks.pm[r0:r0 + nr]

    # ---- triangle multiplication (both directions): channel-parallel contraction --------------------
    # The contraction is independent per channel, so instead of gathering a whole operand on every rank,
    # each rank contracts C/P channels for ALL rows: the producer's channel-major planes are already one
    # contiguous block per destination rank (all-to-all), and the contraction writes its result in groups
    # of output rows, one contiguous block per owner (all-to-all back).  Per rank and direction this moves
    # 3 * (P-1)/P of one local operand instead of (P-1) of them.
    if C_Z % world:
        raise RuntimeError("the sharded triangle multiplication needs the rank count to divide 128 channels")
    cl = C_Z // world                                                                # channels contracted here
    mx = layer.precision == "mxfp8"
    x_send, x_loc = _bf16(world * cl * nr * pn, dev), None
    for incoming in (0, 1):
        w = pk["tri_mul_in" if incoming else "tri_mul_out"]
        # outgoing: planes [D][local row i or j][k], k = all N columns; incoming: [D][column i or j][local row k]
        prow, pcol, pitch = (n, nr, pr) if incoming else (nr, n, pn)
        if mx:
            # MXFP8 on the wire: e4m3 byte planes (half the bytes of bf16) plus their e8m0 scale blocks, both
            # channel-major, so the channel block of every destination rank is contiguous in each
            pitch = (pcol + 15) // 16 * 16
            lib = _lib_handle()
            sf_all, sf_blk = lib.b200pf_mx_scale_bytes(prow, pcol, C_Z), lib.b200pf_mx_scale_bytes(prow, pcol, cl)
            ab_loc = torch.empty(2 * C_Z * prow * pitch, dtype=torch.uint8, device=dev)
            a_loc, b_loc = ab_loc[:C_Z * prow * pitch], ab_loc[C_Z * prow * pitch:]
            sa_loc, sb_loc = (torch.zeros(sf_all, dtype=torch.uint8, device=dev) for _ in range(2))
            call("b200pf_trimul_producer_mx", ptr(z_loc), ptr(mask_loc), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]),
                 ptr(a_loc), ptr(b_loc), ptr(sa_loc), ptr(sb_loc), prow * pitch, pitch, nr, n, incoming, st)
            sa_ch = all_to_all_blocks(sa_loc.view(world, sf_blk), group, "trimul_sa", barrier=False)   # [src][cl][kgroups][row blocks][512]
            sb_ch = all_to_all_blocks(sb_loc.view(world, sf_blk), group, "trimul_sb", barrier=False)
            scales, variant = (ptr(sa_ch), ptr(sb_ch)), 2
        else:
            ab_loc = _bf16(2 * C_Z * prow * pitch, dev)
            a_loc, b_loc = ab_loc[:C_Z * prow * pitch], ab_loc[C_Z * prow * pitch:]
            oa, ob = PlaneOut(ptr(a_loc), prow * pitch, 0, 0), PlaneOut(ptr(b_loc), prow * pitch, 0, 0)
            call("b200pf_trimul_producer", ptr(z_loc), ptr(mask_loc), *ops.trimul_producer_weights(w),
                 C.byref(oa), C.byref(ob), pitch, nr, n, incoming, st)
            scales, variant = (None, None), 0
        # ONE exchange for both operands: block t = (a planes of rank t's channels | b planes of rank t's channels),
        # received as [src][a | b][cl][prow][pitch]; its barrier also covers the scale blocks sent just before
        blk = cl * prow * pitch
        ab_ch = _strided_exchange("trimul_ab", ab_loc, 2 * world * blk, blk, 2, blk, C_Z * prow * pitch, 2 * blk, blk, group)
        if ab_ch is not None:
            a_ch, b_ch, seg = ab_ch, ab_ch[blk:], 2 * blk
        else:
            a_ch = all_to_all_blocks(a_loc.view(world, -1), group, "trimul_a")           # [src][cl][prow][pitch]
            b_ch = all_to_all_blocks(b_loc.view(world, -1), group, "trimul_b")
            seg = blk
        # outgoing: the source rank owns a block of ROWS of the operand; incoming: a block of the contraction index
        pa = Planes(ptr(a_ch), prow * pitch, seg, pitch, prow, pcol, world, incoming)
        pb = Planes(ptr(b_ch), prow * pitch, seg, pitch, prow, pcol, world, incoming)
        call("b200pf_trimul_contract", C.byref(pa), C.byref(pb), *scales, ptr(x_send), nr * pn, pn,
             nr, cl * nr * pn, cl, variant, st)                                     # x[dest][cl][nr][pn]
        x_loc = all_to_all_blocks(x_send.view(world, -1), group, "trimul_x")         # [src = channel block][cl][nr][pn] = [D][nr][pn]
        if side is not None:
            side.before_z_write()          # the previous block's pair-bias projection has read z
        ops.trimul_epilogue(z_loc, x_loc, nr * pn, pn, w, nr, n)
        del ab_loc, a_loc, b_loc, ab_ch, a_ch, b_ch
    del x_send, x_loc

    # ---- triangle attention, starting node (lines = local rows) ---------------------------------
    w = pk["tri_att_start"]
    q, k, v, g, o = (_bf16(nr * n * C_Z, dev) for _ in range(5))
    bias_loc = _bf16(nr * 4 * pn, dev)
    call("b200pf_triatt_producer", ptr(z_loc), *ops.triatt_producer_weights(w), ptr(q), ptr(k), ptr(v), ptr(g),
         ptr(bias_loc), pn, 4 * pn, pn, nr, n, 0, st)
    bias_all = all_gather_cat(bias_loc, group, "tri_bias")                           # [query][head][key]
    call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), pn, ptr(bias_all), pn, 4 * pn, ptr(masks.rows[r0:r0 + nr]),
         masks.pitch, ptr(o), n * C_Z, C_Z, nr, n, st)
    call("b200pf_triatt_epilogue", ptr(z_loc), ptr(o), ptr(g), ptr(w["w_o"]), nr * n, st)

    # ---- triangle attention, ending node (lines = local columns of the column shard) ------------
    w = pk["tri_att_end"]
    zc16 = rows_to_cols_bf16(z_loc, group) if _BF16_EXCHANGE["enabled"] else None
    if zc16 is not None:
        # bf16 on the wire both ways: z goes to the column owners narrowed (the producer rounds its LayerNorm output
        # to bf16 anyway), and only the UPDATE comes back, to be added into the fp32 rows that never moved
        call("b200pf_triatt_producer_bf16z", ptr(zc16), *ops.triatt_producer_weights(w), ptr(q), ptr(k), ptr(v), ptr(g),
             ptr(bias_loc), pn, 4 * pn, pn, n, nr, 1, st)
        bias_all = all_gather_cat(bias_loc, group, "tri_bias")
        call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), pn, ptr(bias_all), pn, 4 * pn, ptr(masks.cols[r0:r0 + nr]),
             masks.pitch, ptr(o), C_Z, nr * C_Z, nr, n, st)
        upd = _bf16(n * nr * C_Z, dev).view(n, nr, C_Z)
        call("b200pf_triatt_epilogue_update", ptr(upd), ptr(o), ptr(g), ptr(w["w_o"]), n * nr, st)
        upd_rows = cols_to_rows(upd, group)                                           # [nr][N][128] bf16
        call("b200pf_add_bf16", ptr(z_loc), ptr(upd_rows), nr * n * C_Z, st)
        del upd, upd_rows
    else:
        zc = rows_to_cols(z_loc, group)                                              # [N][nr][128] fp32
        call("b200pf_triatt_producer", ptr(zc), *ops.triatt_producer_weights(w), ptr(q), ptr(k), ptr(v), ptr(g),
             ptr(bias_loc), pn, 4 * pn, pn, n, nr, 1, st)
        bias_all = all_gather_cat(bias_loc, group, "tri_bias")
        call("b200pf_triatt_core_tc4", ptr(q), ptr(k), ptr(v), pn, ptr(bias_all), pn, 4 * pn, ptr(masks.cols[r0:r0 + nr]),
             masks.pitch, ptr(o), C_Z, nr * C_Z, nr, n, st)
        call("b200pf_triatt_epilogue", ptr(zc), ptr(o), ptr(g), ptr(w["w_o"]), n * nr, st)
        z_loc = cols_to_rows(zc, group)
        del zc
    del q, k, v, g, o, zc16, bias_loc, bias_all

    # ---- pair transition ---------------------------------------------------------------------------
    ops.transition_z_bf16(z_loc, pk["transition_z"])

    # ---- single track: attention for the local query rows, the rest replicated --------------------
    if layer.with_s and s is not None:
        def single_track(channel: int) -> None:
            bias = ops.pair_bias_heads(z_loc, pk["attention"])
            if side is not None:
                side.mark_z_read()
            og_loc = ops.single_track_local(s, z_loc, tok_mask_u8, pk["pre_norm_s"], pk["attention"], pk["s_fused"],
                                            layer.num_heads, r0, bias)
            # output projection and transition are per row: run them on the local rows, then gather s
            s_loc = s[r0:r0 + nr]
            ops.single_track_finish(s_loc, og_loc, pk["attention"], pk["transition_s"], pk["s_fused"])
            s.copy_(all_gather_cat(s_loc, group, "s_rows", channel).view(n, s.shape[1]))

        if side is None:
            single_track(0)
        else:
            z_ready = torch.cuda.Event()
            z_ready.record()
            with torch.cuda.stream(side.stream):
                side.stream.wait_event(z_ready)
                single_track(1)
    return z_loc


class ShardedPairformerModule(nn.Module):
    """Same constructor and forward signature as ``B200PairformerModule``; every rank passes the
    full (replicated) inputs and receives the full outputs, the blocks run row-sharded in between."""

    def __init__(self, token_s: int, token_z: int, num_blocks: int, num_heads: int = 16, dropout: float = 0.25,
                 pairwise_head_width: int = 32, pairwise_num_heads: int = 4, post_layer_norm: bool = False,
                 activation_checkpointing: bool = False, v2: bool = False, precision: str = "bf16", group=None,
                 **kwargs) -> None:
        super().__init__()
        if precision not in ("bf16", "mxfp8"):
            raise NotImplementedError("the sharded trunk is built for the bf16 and mxfp8 tiers")
        self.group = group
        self._side: Optional[SideTrack] = None
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
            side = None
            if z_loc.is_cuda and os.environ.get("B200PF_SIDE_TRACK", "1") != "0":
                if self._side is None or self._side.stream.device != z_loc.device:
                    self._side = SideTrack(z_loc.device)
                side = self._side
            for layer in self.layers:
                z_loc = sharded_block(layer, sw, z_loc, tm, pm, rank, world, self.group, side)
            if side is not None:
                side.join()
            z_loc = z_loc.clone()          # the blocks hand back an exchange's receive buffer, which the next call reuses
        return sw, z_loc

    def forward_rows(self, s: torch.Tensor, z_rows: torch.Tensor, mask: Optional[torch.Tensor] = None,
                     pair_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """The trunk for a caller that keeps z sharded: ``z_rows`` [1, N/P, N, C] are THIS rank's rows (rank r owns
        rows [r N/P, (r+1) N/P)), s [1, N, c_s] and the masks are whole and equal on every rank.  Returns
        (s [1, N, c_s], this rank's rows of z) in the input dtypes; nothing of z is gathered."""
        if not z_rows.is_cuda:
            raise RuntimeError("ShardedPairformerModule: inputs must be CUDA tensors (there is no CPU path)")
        rank = dist.get_rank(self.group)
        z_loc = z_rows[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
        sw, z_loc = self.forward_sharded(s[0], z_loc, mask, pair_mask)
        status = device_status()
        if status:
            raise RuntimeError(f"sharded Pairformer: device status 0x{status:x} on rank {rank} "
                               "(4 = a peer did not reach an exchange barrier in time; 1 = a wait inside a kernel ran out)")
        return sw.unsqueeze(0).to(s.dtype), z_loc.unsqueeze(0).to(z_rows.dtype)

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
        status = device_status()
        if status:
            raise RuntimeError(f"sharded Pairformer: device status 0x{status:x} on rank {rank} "
                               "(4 = a peer did not reach an exchange barrier in time; 1 = a wait inside a kernel ran out)")
        return sw.unsqueeze(0).to(s.dtype), z_out.to(z.dtype)
